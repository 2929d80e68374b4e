"""Torch building blocks shared by the two baseline arms of bench.py (reference endpoint arm, tuned NCCL arm).

Everything here is stock PyTorch: routing, fp8 e4m3 1x128 quantisation, sorting rows by expert, the grouped
SwiGLU expert FFN (``torch.nn.functional.grouped_mm`` when the installed torch has it for this GPU, else one
cuBLAS pair per expert) and the gate-weighted combine (a batched matrix product with fp32 accumulation).
Nothing from the ``dlslime_b200`` package is imported.
"""

from __future__ import annotations

E, TOPK, HIDDEN, INTER = 256, 8, 7168, 2048
FP8_MAX = 448.0


def init_weights(experts, device, seed=0):
    """Same per-expert seeding as the product's ``init_expert_weights``: expert e is drawn from seed*100003+e."""
    import torch

    w13 = torch.empty((len(experts), 2 * INTER, HIDDEN), dtype=torch.bfloat16, device=device)
    w2 = torch.empty((len(experts), HIDDEN, INTER), dtype=torch.bfloat16, device=device)
    gen = torch.Generator(device=device)
    for i, e in enumerate(experts):
        gen.manual_seed(seed * 100003 + e)
        w13[i].copy_(torch.randn((2 * INTER, HIDDEN), generator=gen, device=device).mul_(0.02))
        w2[i].copy_(torch.randn((HIDDEN, INTER), generator=gen, device=device).mul_(0.02))
    return w13, w2


def route(logits):
    import torch

    probs = torch.softmax(logits.float(), dim=-1)
    return torch.topk(probs, TOPK, dim=-1)  # (weights, expert ids)


def quant_1x128(x):
    """bf16 [T, H] -> (e4m3 bytes [T, H], fp32 scales [T, H/128]); the scale arithmetic is fp32 on the small tensor,
    the big tensor is touched once in bf16."""
    import torch

    T = x.shape[0]
    xv = x.view(T, HIDDEN // 128, 128)
    scale = xv.abs().amax(-1).float().clamp_min(1e-4) / FP8_MAX
    q = (xv.float() / scale.unsqueeze(-1)).clamp_(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(T, HIDDEN)
    return q.view(torch.uint8), scale


def dequant_1x128(q_u8, scale):
    """e4m3 bytes [R, H] + scales [R, H/128] -> bf16 [R, H] without an fp32 copy of the rows."""
    import torch

    R = q_u8.shape[0]
    xb = q_u8.view(torch.float8_e4m3fn).to(torch.bfloat16).view(R, HIDDEN // 128, 128)
    return (xb * scale.to(torch.bfloat16).unsqueeze(-1)).view(R, HIDDEN)


class ExpertFFN:
    """Grouped SwiGLU FFN over rows sorted by local expert. ``offs`` = int32 end offsets per expert (device)."""

    def __init__(self, w13, w2):
        import torch

        self.w13, self.w2 = w13, w2
        self.w13_t, self.w2_t = w13.transpose(-2, -1), w2.transpose(-2, -1)
        self.grouped = getattr(torch.nn.functional, "grouped_mm", None) or getattr(torch, "_grouped_mm", None)
        self.mode = "grouped_mm" if self.grouped is not None else "per-expert cuBLAS loop"

    def __call__(self, xd, offs, offs_host=None):
        import torch

        if self.grouped is not None:
            try:
                gu = self.grouped(xd, self.w13_t, offs=offs)
                h = torch.nn.functional.silu(gu[:, :INTER]) * gu[:, INTER:]
                return self.grouped(h, self.w2_t, offs=offs)
            except Exception:  # not available for this device / shape: fall back for the rest of the run
                self.grouped, self.mode = None, "per-expert cuBLAS loop"
        if offs_host is None:
            offs_host = offs.cpu()
        y = torch.empty((xd.shape[0], HIDDEN), dtype=torch.bfloat16, device=xd.device)
        a = 0
        for j in range(self.w13.shape[0]):
            b = int(offs_host[j])
            if b > a:
                gu = xd[a:b] @ self.w13_t[j]
                h = torch.nn.functional.silu(gu[:, :INTER]) * gu[:, INTER:]
                torch.matmul(h, self.w2_t[j], out=y[a:b])
            a = b
        return y


def combine(ret_sorted, order, w, out):
    """ret_sorted: expert outputs of my T*TOPK (token, k) pairs in expert-sorted order; order: the sort permutation."""
    import torch

    T = w.shape[0]
    unsorted = torch.empty_like(ret_sorted)
    unsorted[order] = ret_sorted
    torch.bmm(w.to(torch.bfloat16).unsqueeze(1), unsorted.view(T, TOPK, HIDDEN), out=out.view(T, 1, HIDDEN))
    return out
