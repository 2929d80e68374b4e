"""Guard bands of the symmetric heap: intact after real multi-rank steps, and a stray write is found."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_guard_bands_survive_moe_and_allgather_steps(monkeypatch):
    monkeypatch.setenv("SLIME_HEAP_GUARD", "1")
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig, emulated_forward
    from dlslime_b200.ops.allgather import AllGatherLLBuffer
    from dlslime_b200.ops.ep import EpBuffer

    world, tokens = 4, [9, 0, 33, 64]
    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    bufs = EpBuffer.emulated_group(world, cfg.num_experts, cfg.topk, cfg.hidden, max(tokens))
    heap = bufs[0].heap
    assert heap.guard and len(heap._guards) >= 2
    layers = [ExpertParallelMoE(cfg, max(tokens), buffer=b, seed=3) for b in bufs]
    gen = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(2):
        xs = [torch.randn((t, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16) for t in tokens]
        lgs = [torch.randn((t, cfg.num_experts), generator=gen, device="cuda") for t in tokens]
        emulated_forward(layers, xs, lgs)
    assert heap.check_guards() == []

    group = AllGatherLLBuffer.emulated_group(world, 16, 1024, torch.bfloat16)
    xs = [torch.randn((16, 1024), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(world)]
    for _ in range(3):
        hooks = [g.all_gather_ll_hook(x) for g, x in zip(group, xs)]
        outs = [h() for h in hooks]
    assert torch.equal(outs[-1], torch.cat(xs, dim=0))
    assert group[0].heap.check_guards() == []


def test_stray_write_is_reported(monkeypatch):
    monkeypatch.setenv("SLIME_HEAP_GUARD", "1")
    from dlslime_b200.parallel.symm import GUARD_BYTES, SymmetricHeap

    heap = SymmetricHeap.emulated(2, 1 << 20)
    a = heap.reserve(1000)
    b = heap.reserve(4096)
    assert a == GUARD_BYTES and b >= a + 1000 + GUARD_BYTES
    assert heap.check_guards() == []
    # an overrun of the first reservation (rounded up to 16 bytes) by one byte, in the second rank's region;
    # the byte belongs to this heap, so nothing outside it is touched
    overrun = heap.view(a, (1009,), torch.uint8, rank=1)
    overrun[1008] = 0
    bad = heap.check_guards()
    assert bad == [(1, heap._guards[1])]
    heap.close()


def test_guard_is_off_by_default(monkeypatch):
    monkeypatch.delenv("SLIME_HEAP_GUARD", raising=False)
    from dlslime_b200.parallel.symm import SymmetricHeap

    heap = SymmetricHeap.emulated(1, 1 << 20)
    assert heap.reserve(1000) == 0 and heap.check_guards() == []
    heap.close()
