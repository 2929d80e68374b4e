"""bf16 GEMMs on the tcgen05 tensor cores (``csrc/kernels/gemm.cu``).

Weights use the ``nn.Linear`` layout ``[N, K]`` (K contiguous), activations are
``[M, K]``; accumulation is fp32 in tensor memory, outputs are bf16.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._common import default_status, ptr, require_cuda, stream_ptr

EPI_STORE, EPI_SWIGLU, EPI_SCATTER_ROWS = 0, 1, 2


def _wide_tiles_pay(m: int, n: int, sms: int = 148) -> bool:
    """Whether the 256 x 512 tiling wastes no more of its last wave than the 256-row tilings of width 256 / 224 / 192
    (cost model: waves x (tile width + a per-tile overhead in columns); the wide tiles get 10 % for the power they save)."""
    pairs = max(1, sms // 2)
    mt = -(-m // 256)

    def cost(width, overhead):
        tiles = mt * -(-n // width)
        return -(-tiles // pairs) * (width + overhead)

    return cost(512, 24) <= 1.10 * min(cost(w, 12) for w in (256, 224, 192))


def gemm_bf16_pair(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, wide: bool | None = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ b[N, K].T`` on CTA pairs (256-row tiles, ``tcgen05`` ``cta_group::2``). ``wide``: tiles
    of 256 x 512 (two accumulator blocks share the A tile; less traffic into shared memory per FLOP and an L2-friendly
    tile order), default: where the tile count fits the grid as well as the narrower tilings do."""
    require_cuda(a, b)
    assert a.dtype == b.dtype == torch.bfloat16 and a.stride(1) == 1 and b.stride(1) == 1
    m, k = a.shape
    n, kb = b.shape
    assert k == kb
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if wide is None:
        wide = _wide_tiles_pay(m, n)
    _lib.call("slime_gemm_bf16_wide" if wide else "slime_gemm_bf16_pair", ptr(a), ptr(b), ptr(out), m, n, k, a.stride(0), b.stride(0), out.stride(0),
              default_status().dev_ptr, stream_ptr())
    return out


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, pair: bool | None = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ b[N, K].T``. ``pair`` picks the CTA-pair kernel (default: when M >= 256)."""
    require_cuda(a, b)
    assert a.dtype == b.dtype == torch.bfloat16 and a.stride(1) == 1 and b.stride(1) == 1
    m, k = a.shape
    n, kb = b.shape
    assert k == kb
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if pair is None:
        pair = m >= 256  # two SMs per 256-row tile pay off as soon as there is a full tile
    if pair:
        return gemm_bf16_pair(a, b, out)
    _lib.call("slime_gemm_bf16", ptr(a), ptr(b), ptr(out), m, n, k, a.stride(0), b.stride(0), out.stride(0),
              default_status().dev_ptr, stream_ptr())
    return out


def pick_grouped_tile_n(row_tiles: int, n_out: int, swiglu: bool = False, sms: int = 148) -> int:
    """Tile width (256, 224, 192 or 128 columns of the weight; SwiGLU: half as many output columns) for a grouped GEMM on
    single CTAs that is expected to have ``row_tiles`` 128-row tiles in total: the width whose tile count wastes the least
    of the last wave of the persistent grid (cost = waves x (width + a per-tile overhead in columns); ties go to the wider
    tile). Only for compute-bound launches: a weight-streaming launch (few rows per group) gains nothing from full waves,
    since its CTAs never wait for one another and a short last wave still saturates HBM (measured)."""
    best, best_cost = 256, None
    for width in (256, 224, 192, 128):
        out = width // 2 if swiglu else width
        tiles = max(1, row_tiles) * -(-n_out // out)
        cost = -(-tiles // sms) * (width + 16)
        if best_cost is None or cost < best_cost:
            best, best_cost = width, cost
    return best


def grouped_gemm_bf16(a: torch.Tensor, b: torch.Tensor, group_offsets: torch.Tensor, out: torch.Tensor | None = None,
                      epilogue: int = EPI_STORE, row_info: torch.Tensor | None = None, scatter_bases=None,
                      scatter_row_bytes: int = 0, scatter_slots: int = 0,
                      row_scale: torch.Tensor | None = None, pair: bool | str = False, tile_n: int = 0,
                      w_prefetch: int = 0, tile_m: int = 0) -> torch.Tensor | None:
    """Grouped GEMM over consecutive row groups of ``a``.

    ``a`` is ``[M_cap, K]``; ``group_offsets`` is an int32 device tensor of
    ``G + 1`` row prefixes (rows past ``group_offsets[G]`` are ignored); ``b`` is
    ``[G, N, K]`` (``[G, 2N, K]`` with gate rows before up rows for SwiGLU).
    The group sizes never leave the device, so there is no host synchronisation.

    With ``EPI_SCATTER_ROWS`` nothing is written to ``out``: result row ``r`` is stored at
    ``scatter_bases[info >> 48] + (info & (2**48 - 1)) * scatter_row_bytes`` with
    ``info = row_info[r]`` (int64 device tensor); the regions may live on peer GPUs.

    ``pair`` runs the kernel on CTA pairs (256-row tiles, a third less traffic between L2 and the SMs): the faster form
    for groups of several hundred rows and more, the slower one for small groups (the last tile of a group computes
    up to 255 unused rows instead of up to 127). ``pair="wide"``: CTA pairs with 256 x 512 tiles, another quarter less
    traffic per FLOP, which is what raises the clock under the power limit. ``pair="swap"``: CTA pairs with the operands
    swapped (weight rows on the M side of the MMA, the tokens of a group on the N side in steps of 16): nothing is computed
    for rows that do not exist, and a group of up to 256 rows passes over its weights once. ``tile_n`` (single CTAs only): tile width 128,
    192 or 224 instead of 256, see :func:`pick_grouped_tile_n`. ``w_prefetch`` (single CTAs only): the producer asks L2 for
    the weight boxes this many 64-deep K blocks ahead of its loads, meant for launches that stream weights from HBM (few rows per
    group); measured slower than no prefetch at every distance on this part, so nothing sets it. ``tile_m=64`` (single CTAs, 256-wide
    tiles): row tiles of 64 instead of 128, for groups of a few dozen rows (a decode step): the A part of a pipeline stage
    halves and the ring gets a fifth stage, so more weight bytes are in flight per SM.
    """
    require_cuda(a, b, group_offsets)
    assert a.dtype == b.dtype == torch.bfloat16 and group_offsets.dtype == torch.int32
    assert a.stride(1) == 1 and b.is_contiguous() and b.dim() == 3
    g, rows_b, k = b.shape
    m_cap = a.shape[0]
    n = rows_b // 2 if epilogue == EPI_SWIGLU else rows_b
    assert group_offsets.numel() == g + 1 and a.shape[1] == k
    if epilogue != EPI_SCATTER_ROWS and out is None:
        out = torch.empty((m_cap, n), dtype=torch.bfloat16, device=a.device)
    ldc = out.stride(0) if out is not None else n
    if not pair and (tile_n not in (0, 256) or w_prefetch or tile_m == 64):
        _lib.call("slime_grouped_gemm_bf16_tile", ptr(a), ptr(b), ptr(out), ptr(group_offsets), g, m_cap, n, k, a.stride(0), k, ldc,
                  epilogue, ptr(row_info), scatter_bases, scatter_row_bytes, scatter_slots, ptr(row_scale), int(tile_n), int(w_prefetch), int(tile_m),
                  default_status().dev_ptr, stream_ptr())
        return out
    entry = "slime_grouped_gemm_bf16_swapped" if pair == "swap" else "slime_grouped_gemm_bf16_wide" if pair == "wide" else "slime_grouped_gemm_bf16_pair" if pair else "slime_grouped_gemm_bf16"
    _lib.call(entry, ptr(a), ptr(b), ptr(out),
              ptr(group_offsets), g, m_cap, n, k, a.stride(0), k, ldc, epilogue, ptr(row_info), scatter_bases, scatter_row_bytes, scatter_slots, ptr(row_scale),
              default_status().dev_ptr, stream_ptr())
    return out


def grouped_gemm_bf16_gated(a: torch.Tensor, b: torch.Tensor, group_offsets: torch.Tensor, group_ready: torch.Tensor,
                            *, step: int = 0, step_ptr: int = 0, out: torch.Tensor | None = None,
                            epilogue: int = EPI_STORE, trace: torch.Tensor | None = None,
                            tile_counter: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`grouped_gemm_bf16` (store and SwiGLU epilogues) over groups that are still being filled while the kernel
    runs: the rows of group ``g`` are read once ``group_ready[g] >= step`` (int64 device tensor, one word per group).
    ``step_ptr`` (a device address holding the step number) replaces ``step`` for graph-replayable steps. The kernel
    that fills the rows must be launched first (in front of this one in the stream; this kernel is launched as its
    programmatic dependent). ``trace`` (int64 [G, 2]) receives when the first CTA began to wait for / obtained each group.
    ``tile_counter`` (int32 [2], zeros; the kernel leaves it zero) switches the CTAs from every gridDim-th tile to a
    shared tile counter, which keeps a CTA that shares its SM with the filling kernel from holding the others up."""
    require_cuda(a, b, group_offsets, group_ready)
    assert a.dtype == b.dtype == torch.bfloat16 and group_offsets.dtype == torch.int32 and group_ready.dtype == torch.int64
    assert a.stride(1) == 1 and b.is_contiguous() and b.dim() == 3 and epilogue in (EPI_STORE, EPI_SWIGLU)
    g, rows_b, k = b.shape
    m_cap = a.shape[0]
    n = rows_b // 2 if epilogue == EPI_SWIGLU else rows_b
    assert group_offsets.numel() == g + 1 and a.shape[1] == k and group_ready.numel() >= g
    if out is None:
        out = torch.empty((m_cap, n), dtype=torch.bfloat16, device=a.device)
    _lib.call("slime_grouped_gemm_bf16_gated_traced", ptr(a), ptr(b), ptr(out), ptr(group_offsets), g, m_cap, n, k, a.stride(0), k,
              out.stride(0), epilogue, ptr(group_ready), int(step), step_ptr or None, ptr(trace), ptr(tile_counter),
              default_status().dev_ptr, stream_ptr())
    return out


def grouped_gemm_fp8a(aq: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, group_offsets: torch.Tensor,
                      out: torch.Tensor | None = None, epilogue: int = EPI_STORE) -> torch.Tensor:
    """The grouped GEMM with the activations still in their wire format: ``aq [M_cap, K]`` e4m3 and ``a_scale
    [M_cap, K/128]`` (1x128 scales), bf16 weights ``b [G, N or 2N, K]``. The kernel expands every A tile to bf16 in
    shared memory with the same rounding as :func:`dlslime_b200.ops.quant.fp8_dequant_1x128`, so the result is
    bit-identical to dequantising first and calling :func:`grouped_gemm_bf16`, without the pass over the rows."""
    require_cuda(aq, a_scale, b, group_offsets)
    assert aq.dtype == torch.float8_e4m3fn and b.dtype == torch.bfloat16 and group_offsets.dtype == torch.int32
    assert aq.stride(1) == 1 and b.is_contiguous() and b.dim() == 3 and a_scale.dtype == torch.float32 and a_scale.is_contiguous()
    assert epilogue in (EPI_STORE, EPI_SWIGLU)
    g, rows_b, k = b.shape
    m_cap = aq.shape[0]
    n = rows_b // 2 if epilogue == EPI_SWIGLU else rows_b
    assert group_offsets.numel() == g + 1 and aq.shape[1] == k and k % 128 == 0 and a_scale.shape == (m_cap, k // 128)
    if out is None:
        out = torch.empty((m_cap, n), dtype=torch.bfloat16, device=aq.device)
    _lib.call("slime_grouped_gemm_fp8a", ptr(aq), ptr(a_scale), ptr(b), ptr(out), ptr(group_offsets), g, m_cap, n, k,
              aq.stride(0), k, out.stride(0), epilogue, default_status().dev_ptr, stream_ptr())
    return out


def gemm_fp8_blockscaled(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M, N]`` (bf16) ``= dequant(aq, sa) @ dequant(bq, sb).T`` on the fp8 tensor cores.

    ``aq [M, K]`` / ``bq [N, K]`` are e4m3; ``sa [M, K/128]`` are per-token 1x128 scales, ``sb [ceil(N/128), K/128]``
    128x128 weight-block scales (what :func:`dlslime_b200.ops.quant.fp8_quant_1x128` / ``fp8_quant_128x128`` produce).
    """
    require_cuda(aq, bq, sa, sb)
    assert aq.dtype == bq.dtype == torch.float8_e4m3fn and aq.stride(1) == 1 and bq.stride(1) == 1
    assert sa.dtype == sb.dtype == torch.float32 and sa.is_contiguous() and sb.is_contiguous()
    m, k = aq.shape
    n, kb = bq.shape
    assert k == kb and k % 128 == 0
    assert sa.shape == (m, k // 128) and sb.shape == ((n + 127) // 128, k // 128)
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=aq.device)
    _lib.call("slime_gemm_fp8_blockscaled", ptr(aq), ptr(sa), ptr(bq), ptr(sb), ptr(out), m, n, k, aq.stride(0), bq.stride(0),
              out.stride(0), default_status().dev_ptr, stream_ptr())
    return out


def ref_gemm_fp8_blockscaled(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """fp32 oracle of :func:`gemm_fp8_blockscaled`."""
    m, k = aq.shape
    n = bq.shape[0]
    a = aq.float().view(m, k // 128, 128) * sa.unsqueeze(-1)
    sb_full = sb.repeat_interleave(128, dim=0)[:n]
    b = bq.float().view(n, k // 128, 128) * sb_full.unsqueeze(-1)
    return a.view(m, k) @ b.view(n, k).t()
