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


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ag_gemm_fp8_emulated(world):
    """fp8 payload and scales pushed rank by rank, then the gated block-scaled GEMM of every rank."""
    from dlslime_b200.ops import gemm, quant
    from dlslime_b200.ops.ag_gemm import AllGatherGemmFp8
    from dlslime_b200.ops._common import default_status

    rows, k, n = 256, 512, 256
    group = AllGatherGemmFp8.emulated_group(world, rows, k)
    gen = torch.Generator(device="cuda").manual_seed(19)
    ws = [quant.fp8_quant_128x128((torch.randn((n, k), generator=gen, device="cuda") * 0.05).to(torch.bfloat16)) for _ in range(world)]
    for step in (1, 2):
        xs = [quant.fp8_quant_1x128(torch.randn((rows, k), generator=gen, device="cuda").to(torch.bfloat16)) for _ in range(world)]
        outs = [torch.empty((world * rows, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for g, (xq, sx) in zip(group, xs):
            g.push(xq, sx, step)
        for g, (wq, sb), o in zip(group, ws, outs):
            g.gemm(wq, sb, o, step)
        torch.cuda.synchronize()
        default_status().check()
        fq = torch.cat([x[0].view(torch.uint8) for x in xs], 0)
        fs = torch.cat([x[1] for x in xs], 0)
        for r, (g, (wq, sb), o) in enumerate(zip(group, ws, outs)):
            gq, gs = g.gathered
            assert torch.equal(gq.view(torch.uint8), fq) and torch.equal(gs, fs), "gathered payload or scales differ"
            ref = gemm.ref_gemm_fp8_blockscaled(fq.view(torch.float8_e4m3fn), fs, wq, sb)
            err = (o.float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-3, f"rank {r}: {err}"


def test_ag_gemm_fp8_single_rank_fused():
    from dlslime_b200.ops import quant
    from dlslime_b200.ops.ag_gemm import AllGatherGemmFp8
    from dlslime_b200.ops._common import default_status

    rows, k, n = 384, 1024, 512
    g = AllGatherGemmFp8.emulated_group(1, rows, k)[0]
    x = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    wq, sb = quant.fp8_quant_128x128(w)
    for _ in range(2):
        out = g(x, wq, sb)
        torch.cuda.synchronize()
        default_status().check()
        ref = x.float() @ w.float().t()
        rel = (out.float() - ref).norm() / ref.norm()
        assert rel < 0.08, rel.item()
