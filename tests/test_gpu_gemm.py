"""tcgen05 GEMM kernels against an fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(out, ref, k):
    # bf16 output of an fp32 accumulation: relative 2^-7 of the result magnitude plus a
    # small absolute term for cancellation
    err = (out.float() - ref).abs()
    tol = ref.abs() * 2 ** -7 + 2 ** -7 * ref.abs().mean() + 1e-3
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad} of {out.numel()} elements off; max err {err.max().item():.4g}"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 4096), (1000, 4096, 4096), (77, 96, 136),
                                   (8192, 3584, 512), (4096, 1152, 256), (300, 4128, 192)])  # tile widths 224 and 192, ragged last tile
def test_gemm_bf16(m, n, k):
    from dlslime_b200.ops import gemm
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.gemm_bf16(a, b, pair=False)
    torch.cuda.synchronize()
    default_status().check()
    ref = a.float() @ b.float().t()
    _check(out, ref, k)


@pytest.mark.parametrize("pair", [False, True, "wide", "swap"])
def test_grouped_gemm_store_and_swiglu(pair):
    from dlslime_b200.ops import gemm
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(5)
    sizes = [0, 5, 128, 131, 300, 1, 0, 64] + ([256, 700, 513] if pair else [])
    g, k, n = len(sizes), 512, 256
    offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    total = sum(sizes)
    a = torch.randn(total + 50, k, device="cuda", dtype=torch.bfloat16)  # extra rows past the last group are ignored
    w = (torch.randn(g, n, k, device="cuda") * 0.05).to(torch.bfloat16)
    out = torch.full((total + 50, n), 7.0, device="cuda", dtype=torch.bfloat16)
    gemm.grouped_gemm_bf16(a, w, offs, out=out, pair=pair)
    torch.cuda.synchronize()
    default_status().check()
    start = 0
    for gi, sz in enumerate(sizes):
        if sz:
            ref = a[start:start + sz].float() @ w[gi].float().t()
            _check(out[start:start + sz], ref, k)
        start += sz
    assert (out[total:] == 7.0).all(), "rows outside every group must not be written"

    # SwiGLU: weights hold N gate rows then N up rows per group
    n_int = 128
    w2 = (torch.randn(g, 2 * n_int, k, device="cuda") * 0.05).to(torch.bfloat16)
    h = gemm.grouped_gemm_bf16(a, w2, offs, epilogue=gemm.EPI_SWIGLU, pair=pair)
    torch.cuda.synchronize()
    default_status().check()
    start = 0
    for gi, sz in enumerate(sizes):
        if sz:
            x = a[start:start + sz].float()
            gate = x @ w2[gi, :n_int].float().t()
            up = x @ w2[gi, n_int:].float().t()
            _check(h[start:start + sz], torch.nn.functional.silu(gate) * up, k)
        start += sz


@pytest.mark.parametrize("tile_n,w_prefetch,tile_m", [(128, 0, 0), (192, 3, 0), (224, 0, 0), (0, 4, 0), (0, 40, 0), (0, 0, 64)])
def test_grouped_gemm_narrow_tiles(tile_n, w_prefetch, tile_m):
    """The single-CTA grouped GEMM with tile widths other than 256, with the weight prefetch into L2 (a distance
    shorter and longer than the K loop of 6 blocks) and with row tiles of 64: store, SwiGLU (an output width that the
    half tile does not divide) and scatter epilogues against the fp32 product."""
    import ctypes

    from dlslime_b200.ops import gemm
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(tile_n + w_prefetch + tile_m)
    sizes = [3, 0, 130, 257, 64]
    g, k, n = len(sizes), 384, 448
    total = sum(sizes)
    offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    a = torch.randn(total, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(g, n, k, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(g, 2 * n, k, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.grouped_gemm_bf16(a, w, offs, tile_n=tile_n, w_prefetch=w_prefetch, tile_m=tile_m)
    h = gemm.grouped_gemm_bf16(a, w2, offs, epilogue=gemm.EPI_SWIGLU, tile_n=tile_n, w_prefetch=w_prefetch, tile_m=tile_m)
    dst = torch.zeros(total, n, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(total, device="cuda")
    bases = (ctypes.c_ulonglong * 8)()
    bases[0] = dst.data_ptr()
    gemm.grouped_gemm_bf16(a, w, offs, epilogue=gemm.EPI_SCATTER_ROWS, row_info=perm.to(torch.int64), scatter_bases=bases,
                           scatter_row_bytes=n * 2, scatter_slots=total, tile_n=tile_n, w_prefetch=w_prefetch, tile_m=tile_m)
    torch.cuda.synchronize()
    default_status().check()
    start = 0
    for gi, sz in enumerate(sizes):
        if sz:
            x = a[start:start + sz].float()
            ref = x @ w[gi].float().t()
            _check(out[start:start + sz], ref, k)
            _check(dst[perm[start:start + sz]], ref, k)
            _check(h[start:start + sz], torch.nn.functional.silu(x @ w2[gi, :n].float().t()) * (x @ w2[gi, n:].float().t()), k)
        start += sz


@pytest.mark.parametrize("pair", [False, True, "wide", "swap"])
def test_grouped_gemm_scatter_rows(pair):
    from dlslime_b200.ops import gemm
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(6)
    sizes = [40, 0, 200] + ([517] if pair else [])
    g, k, n = len(sizes), 256, 512
    total = sum(sizes)
    offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    a = torch.randn(total, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(g, n, k, device="cuda") * 0.05).to(torch.bfloat16)
    dst = torch.zeros(total, n, device="cuda", dtype=torch.bfloat16)
    perm = torch.randperm(total, device="cuda")
    import ctypes

    row_info = perm.to(torch.int64).clone()  # region 0, slot = destination row
    row_info[3] = -1  # dropped row (region index out of range)
    bases = (ctypes.c_ulonglong * 8)()
    bases[0] = dst.data_ptr()
    scale = torch.rand(total, device="cuda") + 0.5
    gemm.grouped_gemm_bf16(a, w, offs, epilogue=gemm.EPI_SCATTER_ROWS, row_info=row_info, scatter_bases=bases,
                           scatter_row_bytes=n * 2, scatter_slots=total, row_scale=scale, pair=pair)
    torch.cuda.synchronize()
    default_status().check()
    ref = torch.zeros(total, n, device="cuda")
    start = 0
    for gi, sz in enumerate(sizes):
        if sz:
            ref[start:start + sz] = (a[start:start + sz].float() @ w[gi].float().t()) * scale[start:start + sz, None]
        start += sz
    expect = torch.zeros_like(ref)
    expect[perm] = ref
    expect[perm[3]] = 0
    _check(dst, expect, k)


@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 512, 512), (1000, 4096, 4096), (8192, 3584, 512), (4096, 1152, 256), (300, 4128, 192),
                                   (2048, 8192, 8192)])
def test_gemm_bf16_cta_pair(m, n, k, wide):
    """The cta_group::2 kernels (256-row tiles on two SMs; ``wide``: 256 x 512 tiles in two accumulator blocks): same
    product, ragged edges in M and N (a tile whose second block lies outside N), all tile widths, several bands of
    tile columns (the last one narrower)."""
    from dlslime_b200.ops import gemm
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(m + n + k + 1)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    out = gemm.gemm_bf16_pair(a, b, wide=wide)
    torch.cuda.synchronize()
    default_status().check()
    ref = a.float() @ b.float().t()
    _check(out, ref, k)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 1024), (1000, 3584, 2048), (300, 4128, 512)])
def test_gemm_fp8_blockscaled(m, n, k):
    """e4m3 x e4m3 with 1x128 activation scales and 128x128 weight scales against the fp32 product of the dequantised operands."""
    from dlslime_b200.ops import gemm, quant
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(m * 3 + n + k)
    a = (torch.randn(m, k, device="cuda") * torch.rand(m, 1, device="cuda") * 4).to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    aq, sa = quant.fp8_quant_1x128(a)
    wq, sb = quant.fp8_quant_128x128(w)
    out = gemm.gemm_fp8_blockscaled(aq, sa, wq, sb)
    torch.cuda.synchronize()
    default_status().check()
    ref = gemm.ref_gemm_fp8_blockscaled(aq, sa, wq, sb)
    # same quantised operands on both sides: only fp32 summation order and the bf16 rounding of the output differ
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3, err
    # and the product is a faithful fp8 approximation of the bf16 one
    full = a.float() @ w.float().t()
    rel = (out.float() - full).norm() / full.norm()
    assert rel < 0.08, rel.item()


def test_grouped_gemm_with_fp8_activations_is_bit_identical_to_dequant_then_gemm():
    """The gate/up GEMM fed with e4m3 rows and 1x128 scales (expanded in shared memory) against the two-pass path."""
    from dlslime_b200.ops import gemm, quant
    from dlslime_b200.ops._common import default_status

    torch.manual_seed(11)
    sizes = [0, 5, 128, 131, 300, 1, 0, 64]
    g, k, inter = len(sizes), 1024, 256
    offs = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device="cuda")
    total = sum(sizes)
    x = (torch.randn(total + 37, k, device="cuda") * torch.rand(total + 37, 1, device="cuda") * 3).to(torch.bfloat16)
    xq, xs = quant.fp8_quant_1x128(x)
    xd = quant.fp8_dequant_1x128(xq, xs)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.05).to(torch.bfloat16)
    w = (torch.randn(g, inter, k, device="cuda") * 0.05).to(torch.bfloat16)
    for weights, epi in ((w13, gemm.EPI_SWIGLU), (w, gemm.EPI_STORE)):
        ref = torch.zeros((total + 37, inter), device="cuda", dtype=torch.bfloat16)
        out = torch.zeros_like(ref)
        gemm.grouped_gemm_bf16(xd, weights, offs, out=ref, epilogue=epi)
        gemm.grouped_gemm_fp8a(xq, xs, weights, offs, out=out, epilogue=epi)
        torch.cuda.synchronize()
        default_status().check()
        assert torch.equal(out[:total], ref[:total]), (out[:total].float() - ref[:total].float()).abs().max().item()
        assert bool((out[total:] == 0).all())
