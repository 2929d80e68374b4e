#!/usr/bin/env python
"""Single-GPU micro-benchmarks of the sm_100a kernels against their library baselines.

    python bench/kernel_bench.py gemm [--m 8192 --n 8192 --k 8192]
    python bench/kernel_bench.py gemm_fp8 [--m 8192 --n 8192 --k 8192]   # e4m3, 1x128 / 128x128 block scales
    python bench/kernel_bench.py grouped [--experts 32 --rows 1024]
    python bench/kernel_bench.py quant

Timing: CUDA events on the launching stream, 3 warm-up runs, a 256 MB buffer is
rewritten between timed runs to flush L2, best and median of the timed runs are
reported. Fractions are of the measured peaks in MEASURED_PEAKS.json when that
file is present (else of 6.65 TB/s and 1.59 PFLOP/s, an earlier measurement).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


_flush = None


def timeit(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        _flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[0], times[len(times) // 2]


_sampler = None


def sustained(fn, flops, secs=1.5):
    """The same kernel back to back for ``secs`` seconds (no L2 flush: the operands are larger than L2), with the SM
    clock and board power sampled meanwhile: a large GEMM runs against the power limit, so what a kernel sustains is
    set by the energy it needs per FLOP, and the burst figure of a single launch does not show it.
    ``tensor_eff_at_clock`` = FLOP/s / (SMs x 8192 FLOP/clk x median SM clock)."""
    global _sampler
    import importlib.util
    import time

    if _sampler is None:
        spec = importlib.util.spec_from_file_location("_root_bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _sampler = mod.ClockSampler(torch.cuda.current_device())
        time.sleep(0.3)
    for _ in range(3):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); fn(); e1.record(); torch.cuda.synchronize()
    n = max(10, int(secs * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
    t0 = time.time()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    ms = e0.elapsed_time(e1) / n
    w = _sampler.window(t0 + 0.3 * (t1 - t0), t1)  # the clock has settled after the first third
    clk = w.get("sm_mhz") or 0
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    time.sleep(0.5)
    return {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "sm_mhz": clk, "power_w_max": w.get("power_w_max"),
            "reasons": w.get("reasons"), "tensor_eff_at_clock": round(flops / (ms * 1e-3) / (sms * 8192 * clk * 1e6), 3) if clk else None}


def cmd_gemm(a):
    from dlslime_b200.ops import gemm

    hbm, tf, tag = peaks()
    x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * a.m * a.n * a.k
    best, med = timeit(lambda: gemm.gemm_bf16(x, w, out=out, pair=False), a.iters)
    b2, m2 = timeit(lambda: torch.matmul(x, w.t(), out=out), a.iters)
    bp, mp = timeit(lambda: gemm.gemm_bf16_pair(x, w, out=out, wide=False), a.iters)
    bw, mw = timeit(lambda: gemm.gemm_bf16_pair(x, w, out=out, wide=True), a.iters)
    extra = {}
    if a.sustained:
        extra["sustained"] = {"cublas": sustained(lambda: torch.matmul(x, w.t(), out=out), flops),
                              "pair_wide": sustained(lambda: gemm.gemm_bf16_pair(x, w, out=out, wide=True), flops),
                              "pair": sustained(lambda: gemm.gemm_bf16_pair(x, w, out=out, wide=False), flops),
                              "cublas_again": sustained(lambda: torch.matmul(x, w.t(), out=out), flops)}
    print(json.dumps({"kernel": "gemm_bf16_tc", "m": a.m, "n": a.n, "k": a.k, "ms_best": round(best, 4), "ms_median": round(med, 4),
                      "wide_ms_best": round(bw, 4), "wide_ms_median": round(mw, 4), "wide_tflops_best": round(flops / bw / 1e9, 1),
                      "wide_frac_of_peak": round(flops / bw / 1e9 / tf, 3), "auto_picks_wide": gemm._wide_tiles_pay(a.m, a.n), **extra,
                      "tflops_best": round(flops / best / 1e9, 1), "frac_of_peak": round(flops / best / 1e9 / tf, 3), "peak": tag,
                      "pair_ms_best": round(bp, 4), "pair_ms_median": round(mp, 4), "pair_tflops_best": round(flops / bp / 1e9, 1),
                      "pair_frac_of_peak": round(flops / bp / 1e9 / tf, 3),
                      "cublas_ms_best": round(b2, 4), "cublas_tflops_best": round(flops / b2 / 1e9, 1)}))
    if _sampler is not None:
        _sampler.stop()


def cmd_gemm_fp8(a):
    from dlslime_b200.ops import gemm, quant

    hbm, tf, tag = peaks()
    x = torch.randn(a.m, a.k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(a.n, a.k, device="cuda") * 0.02).to(torch.bfloat16)
    xq, sx = quant.fp8_quant_1x128(x)
    wq, sw = quant.fp8_quant_128x128(w)
    out = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * a.m * a.n * a.k
    best, med = timeit(lambda: gemm.gemm_fp8_blockscaled(xq, sx, wq, sw, out=out), a.iters)
    b2, _ = timeit(lambda: gemm.gemm_bf16(x, w, out=out), a.iters)
    print(json.dumps({"kernel": "gemm_fp8_blockscaled", "m": a.m, "n": a.n, "k": a.k, "ms_best": round(best, 4), "ms_median": round(med, 4),
                      "tflops_best": round(flops / best / 1e9, 1), "vs_measured_bf16_peak": round(flops / best / 1e9 / tf, 3), "peak": tag,
                      "bf16_pair_kernel_ms_best": round(b2, 4)}))


def cmd_grouped(a):
    from dlslime_b200.ops import gemm

    hbm, tf, tag = peaks()
    g, rows, k, inter = a.experts, a.rows, 7168, 2048
    if a.ragged:  # group sizes as a uniform router produces them: multinomial around the mean, same total
        gen = torch.Generator().manual_seed(0)
        sizes = torch.bincount(torch.randint(0, g, (g * rows,), generator=gen), minlength=g)
        offs = torch.cat([torch.zeros(1, dtype=torch.long), sizes.cumsum(0)]).to(torch.int32).cuda()
    else:
        offs = torch.arange(0, g + 1, dtype=torch.int32, device="cuda") * rows
    x = torch.randn(g * rows, k, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(g, k, inter, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(g * rows, inter, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(g * rows, k, device="cuda", dtype=torch.bfloat16)
    f1, f2 = 2.0 * g * rows * k * 2 * inter, 2.0 * g * rows * inter * k
    b1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU), a.iters)
    b2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y), a.iters)
    p1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair=True), a.iters)
    p2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair=True), a.iters)
    q1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair="wide"), a.iters)
    q2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair="wide"), a.iters)
    s1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair="swap"), a.iters)
    s2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair="swap"), a.iters)

    extra = {}
    row_tiles = int(((offs[1:] - offs[:-1] + 127) // 128).sum().item())
    t1, t2 = gemm.pick_grouped_tile_n(row_tiles, inter, swiglu=True), gemm.pick_grouped_tile_n(row_tiles, k)
    if (t1, t2) != (256, 256):  # few tiles: the width that fills the waves of the grid
        n1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, tile_n=t1), a.iters)
        n2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, tile_n=t2), a.iters)
        wbytes = (w13.numel() + w2.numel()) * 2
        extra["picked_tile_n"] = {"gate_up": t1, "down": t2, "gate_up_ms": round(n1, 4), "down_ms": round(n2, 4),
                                  "weights_tbs": round(wbytes / (n1 + n2) / 1e9, 2), "weights_tbs_tile_256": round(wbytes / (b1 + b2) / 1e9, 2)}
    if rows <= 48:  # groups of a few dozen rows: row tiles of 64 and a fifth pipeline stage
        m1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, tile_m=64), a.iters)
        m2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, tile_m=64), a.iters)
        wbytes = (w13.numel() + w2.numel()) * 2
        extra["tile_m_64"] = {"gate_up_ms": round(m1, 4), "down_ms": round(m2, 4), "weights_tbs": round(wbytes / (m1 + m2) / 1e9, 2),
                              "weights_tbs_tile_m_128": round(wbytes / (b1 + b2) / 1e9, 2)}
    if a.prefetch:  # weight prefetch into L2, for the weight-streaming shapes
        extra["w_prefetch"] = {}
        wbytes = (w13.numel() + w2.numel()) * 2
        for d in (4, 8, 16, 32):
            n1, _ = timeit(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, w_prefetch=d), a.iters)
            n2, _ = timeit(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, w_prefetch=d), a.iters)
            extra["w_prefetch"][d] = {"gate_up_ms": round(n1, 4), "down_ms": round(n2, 4), "weights_tbs": round(wbytes / (n1 + n2) / 1e9, 2)}
        extra["w_prefetch"][0] = {"gate_up_ms": round(b1, 4), "down_ms": round(b2, 4), "weights_tbs": round(wbytes / (b1 + b2) / 1e9, 2)}
    if a.sustained:
        extra["sustained_gate_up"] = {
            "single": sustained(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU), f1),
            "pair": sustained(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair=True), f1),
            "wide": sustained(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair="wide"), f1),
            "swap": sustained(lambda: gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair="swap"), f1)}
        extra["sustained_down"] = {
            "single": sustained(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y), f2),
            "pair": sustained(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair=True), f2),
            "wide": sustained(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair="wide"), f2),
            "swap": sustained(lambda: gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair="swap"), f2)}

    def cublas_loop():
        for e in range(g):
            gu = x[e * rows:(e + 1) * rows] @ w13[e].t()
            hh = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
            torch.matmul(hh, w2[e].t(), out=y[e * rows:(e + 1) * rows])

    b3, _ = timeit(cublas_loop, max(3, a.iters // 2))
    print(json.dumps({"kernel": "grouped_swiglu_ffn", "experts": g, "rows_per_expert": rows, "ragged": bool(a.ragged),
                      "pair_gate_up_ms": round(p1, 4), "pair_gate_up_tflops": round(f1 / p1 / 1e9, 1),
                      "pair_down_ms": round(p2, 4), "pair_down_tflops": round(f2 / p2 / 1e9, 1),
                      "pair_frac_of_peak": round((f1 + f2) / (p1 + p2) / 1e9 / tf, 3),
                      "swap_gate_up_ms": round(s1, 4), "swap_gate_up_tflops": round(f1 / s1 / 1e9, 1),
                      "swap_down_ms": round(s2, 4), "swap_down_tflops": round(f2 / s2 / 1e9, 1),
                      "swap_frac_of_peak": round((f1 + f2) / (s1 + s2) / 1e9 / tf, 3),
                      "wide_gate_up_ms": round(q1, 4), "wide_gate_up_tflops": round(f1 / q1 / 1e9, 1),
                      "wide_down_ms": round(q2, 4), "wide_down_tflops": round(f2 / q2 / 1e9, 1),
                      "wide_frac_of_peak": round((f1 + f2) / (q1 + q2) / 1e9 / tf, 3),
                      "gate_up_ms": round(b1, 4), "gate_up_tflops": round(f1 / b1 / 1e9, 1),
                      "down_ms": round(b2, 4), "down_tflops": round(f2 / b2 / 1e9, 1),
                      "frac_of_peak": round((f1 + f2) / (b1 + b2) / 1e9 / tf, 3), "peak": tag,
                      "cublas_loop_ms": round(b3, 4), "cublas_loop_tflops": round((f1 + f2) / b3 / 1e9, 1), **extra}))
    if _sampler is not None:
        _sampler.stop()


def cmd_quant(a):
    from dlslime_b200.ops import quant

    hbm, tf, tag = peaks()
    x = torch.randn(a.rows_q, 7168, device="cuda").to(torch.bfloat16)
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    s = torch.empty(a.rows_q, 56, device="cuda")
    y = torch.empty_like(x)
    nbytes_q = x.numel() * 3 + s.numel() * 4
    b1, _ = timeit(lambda: quant.fp8_quant_1x128(x, q, s), a.iters)
    b2, _ = timeit(lambda: quant.fp8_dequant_1x128(q, s, y), a.iters)
    b3, _ = timeit(lambda: quant.ref_quant_1x128(x), a.iters)
    print(json.dumps({"kernel": "fp8_quant_1x128", "rows": a.rows_q, "quant_ms": round(b1, 4), "quant_gbs": round(nbytes_q / b1 / 1e6, 1),
                      "dequant_ms": round(b2, 4), "dequant_gbs": round(nbytes_q / b2 / 1e6, 1),
                      "frac_of_peak": round(nbytes_q / b1 / 1e6 / hbm, 3), "peak": tag, "torch_composite_ms": round(b3, 4)}))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["gemm", "gemm_fp8", "grouped", "quant"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--sustained", action="store_true", help="gemm, grouped: also loop each kernel for seconds and sample clock and power")
    ap.add_argument("--prefetch", action="store_true", help="grouped: also time the single-CTA kernels with the weight prefetch into L2")
    ap.add_argument("--ragged", action="store_true", help="grouped: multinomial group sizes instead of equal ones")
    ap.add_argument("--rows-q", type=int, default=32768)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    {"gemm": cmd_gemm, "gemm_fp8": cmd_gemm_fp8, "grouped": cmd_grouped, "quant": cmd_quant}[args.cmd](args)
