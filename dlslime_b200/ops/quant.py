"""Block-scaled fp8 e4m3 quantisation (1x128 activations, 128x128 weights).

With c = max(amax, 1e-4) in fp32: scale = c / 448 and q = rne_sat(x * (448 / c)), i.e. two IEEE divisions
per block and one multiply per element; round-to-nearest-even, saturating.
The kernels are ``csrc/kernels/fp8_quant.cu``; the PyTorch functions below
restate the same arithmetic in fp32 and are the oracle the tests compare against.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._common import ptr, require_cuda, stream_ptr

FP8_MAX = 448.0
AMAX_FLOOR = 1e-4


def fp8_quant_1x128(x: torch.Tensor, out: torch.Tensor | None = None, scales: torch.Tensor | None = None):
    """bf16 [R, H] -> (e4m3 [R, H], fp32 scales [R, H/128])."""
    require_cuda(x)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    if scales is None:
        scales = torch.empty((rows, cols // 128), dtype=torch.float32, device=x.device)
    _lib.call("slime_fp8_quant_1x128", ptr(x), ptr(out), ptr(scales), rows, cols, x.stride(0), out.stride(0), stream_ptr())
    return out, scales


def fp8_dequant_1x128(q: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None, rows: int | None = None):
    """(e4m3 [R, H], fp32 [R, H/128]) -> bf16 [R, H]."""
    require_cuda(q, scales)
    assert q.dim() == 2 and q.stride(1) == 1 and scales.is_contiguous()
    r, cols = q.shape
    if rows is not None:
        r = rows
    if out is None:
        out = torch.empty((q.shape[0], cols), dtype=torch.bfloat16, device=q.device)
    _lib.call("slime_fp8_dequant_1x128", ptr(q), ptr(scales), ptr(out), r, cols, q.stride(0), out.stride(0), stream_ptr())
    return out


def fp8_quant_128x128(w: torch.Tensor):
    """bf16 [N, K] -> (e4m3 [N, K], fp32 scales [ceil(N/128), ceil(K/128)])."""
    require_cuda(w)
    assert w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1
    rows, cols = w.shape
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=w.device)
    scales = torch.empty(((rows + 127) // 128, (cols + 127) // 128), dtype=torch.float32, device=w.device)
    _lib.call("slime_fp8_quant_128x128", ptr(w), ptr(q), ptr(scales), rows, cols, w.stride(0), q.stride(0), stream_ptr())
    return q, scales


# ---------------------------------------------------------------------------
# PyTorch restatements (oracles; run on CPU or GPU)
# ---------------------------------------------------------------------------
def ref_quant_1x128(x: torch.Tensor):
    xf = x.float().reshape(x.shape[0], -1, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(AMAX_FLOOR)
    # tensor / tensor: IEEE divisions, once per group; elements are then multiplied, exactly as the kernels do
    scale = amax / torch.full_like(amax, FP8_MAX)
    inv = torch.full_like(amax, FP8_MAX) / amax
    q = (xf * inv.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), scale


def ref_dequant_1x128(q: torch.Tensor, scale: torch.Tensor):
    qf = q.float().reshape(q.shape[0], -1, 128)
    return (qf * scale.unsqueeze(-1)).reshape(q.shape)


def ref_quant_128x128(w: torch.Tensor):
    rows, cols = w.shape
    pr, pc = (rows + 127) // 128 * 128, (cols + 127) // 128 * 128
    wf = torch.zeros((pr, pc), dtype=torch.float32, device=w.device)
    wf[:rows, :cols] = w.float()
    blocks = wf.reshape(pr // 128, 128, pc // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(AMAX_FLOOR)
    scale = amax / torch.full_like(amax, FP8_MAX)
    inv = torch.full_like(amax, FP8_MAX) / amax
    q = (blocks * inv[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(pr, pc)[:rows, :cols].contiguous(), scale
