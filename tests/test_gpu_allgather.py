"""Low-latency all-gather buffer on one GPU: every rank of an emulated group pushes, then every rank waits.

The ranks share one device, so a push never waits for a peer inside its own launch (the hook form);
the waits run afterwards, when every flag they poll has already been published.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_gather_ll_emulated_group(world):
    from dlslime_b200.ops.allgather import AllGatherLLBuffer

    hidden = 7168
    group = AllGatherLLBuffer.emulated_group(world, 128, hidden, torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(5)
    for bs in [1, 16, 128, 16, 1]:  # both halves of the double buffer are reused
        xs = [torch.randn((bs, hidden), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(world)]
        hooks = [g.all_gather_ll_hook(x) for g, x in zip(group, xs)]
        outs = [h() for h in hooks]
        torch.cuda.synchronize()
        group[0].status.check()
        ref = torch.cat(xs, dim=0)
        for r, out in enumerate(outs):
            assert out.shape == (world * bs, hidden)
            assert torch.equal(out, ref), f"rank {r} bs={bs}: gathered rows differ"


def test_all_gather_ll_rejects_bad_input():
    from dlslime_b200.ops.allgather import AllGatherLLBuffer

    g = AllGatherLLBuffer.emulated_group(2, 4, 256, torch.bfloat16)[0]
    with pytest.raises(ValueError):
        g.all_gather_ll_hook(torch.zeros((8, 256), dtype=torch.bfloat16, device="cuda"))  # more rows than max_bs
    with pytest.raises(ValueError):
        g.all_gather_ll_hook(torch.zeros((2, 256), dtype=torch.float32, device="cuda"))  # wrong dtype
