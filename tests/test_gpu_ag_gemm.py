"""All-gather -> GEMM, replayed rank by rank on one GPU (two-kernel form)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ag_gemm_emulated(world):
    from dlslime_b200.ops.ag_gemm import AllGatherGemm
    from dlslime_b200.ops._common import default_status

    rows, k, n = 256, 512, 256
    group = AllGatherGemm.emulated_group(world, rows, k)
    gen = torch.Generator(device="cuda").manual_seed(9)
    ws = [(torch.randn((n, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(world)]
    for step in (1, 2):
        xs = [torch.randn((rows, k), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(world)]
        outs = [torch.empty((world * rows, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for g, x in zip(group, xs):
            g.push(x, step)
        for g, w, o in zip(group, ws, outs):
            g.gemm(w, o, step)
        torch.cuda.synchronize()
        default_status().check()
        full = torch.cat(xs, 0)
        for r, (g, w, o) in enumerate(zip(group, ws, outs)):
            assert torch.equal(g.gathered, full), "gathered activations differ"
            ref = full.float() @ w.float().t()
            err = (o.float() - ref).abs()
            assert (err <= ref.abs() * 2 ** -7 + ref.abs().mean() * 2 ** -7 + 1e-3).all(), f"rank {r}: {err.max().item()}"


def test_ag_gemm_single_rank_fused():
    from dlslime_b200.ops.ag_gemm import AllGatherGemm
    from dlslime_b200.ops._common import default_status

    rows, k, n = 384, 1024, 512
    g = AllGatherGemm.emulated_group(1, rows, k)[0]
    x = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    for _ in range(2):
        out = g(x, w)
        torch.cuda.synchronize()
        default_status().check()
        ref = x.float() @ w.float().t()
        assert ((out.float() - ref).abs() <= ref.abs() * 2 ** -7 + ref.abs().mean() * 2 ** -7 + 1e-3).all()
