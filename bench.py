#!/usr/bin/env python
"""Headline benchmark: DeepSeek-V3-shaped expert-parallel MoE dispatch + combine.

    python bench.py --gpus N --steps K --warmup W [--mode ll|normal] [--impl ours|reference]

One step is a full MoE layer forward on every rank: top-8 routing of T tokens
over 256 experts, dispatch with fp8 e4m3 1x128 quantisation, the grouped SwiGLU
expert FFN (hidden 7168, intermediate 2048, bf16 weights N(0, 0.02)) and the
gate-weighted bf16 combine. ``--mode ll`` uses T = 128 tokens per rank (decode),
``--mode normal`` T = 4096 (prefill). Inputs are synthetic and seeded, weights
random-init. Timing is CUDA events on the launching stream, max over ranks,
after warm-up, bracketed by a barrier and a device synchronise.

The line printed by rank 0 reports the step latency in microseconds (the whole
layer, nothing skipped), the end-to-end figure through the public API including
the pinned host->device copy of the step's inputs and the device->host read of
its output, aggregate tokens/s, the NVLink payload rate per rank, and the SM
clocks sampled during the timed region.

``--impl reference`` runs the same workload with the unmodified reference package
installed under ``baseline/_ref``: its ``NVLinkEndpoint.read`` moves the token
rows (the only NVLink path it has), NCCL carries the counts, and torch / cuBLAS do
the quantisation, expert FFN and weighted sum, the way a user of the reference
would compose them.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E, TOPK, HIDDEN, INTER = 256, 8, 7168, 2048
T_MODE = {"ll": 128, "normal": 4096}


# ---------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.t0 = self.t1 = None

    def mark_begin(self):
        """The timed region starts now (the sampler may have been started earlier, e.g. before the warm-up)."""
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu=timestamp,{self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 10:
                    continue
                try:
                    import datetime

                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                except ValueError:
                    ts = None
                rows.append((ts, parts[1:]))
        # samples taken inside the marked window; if the marks are missing or nothing falls inside, all of them
        inside = [r for r in rows if r[0] is not None and self.t0 is not None and self.t1 is not None and self.t0 <= r[0] <= self.t1 + 0.05]
        for _, parts in (inside or rows):
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------
# distributed plumbing
# ---------------------------------------------------------------------------------
def init_dist(n_gpus: int):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            # re-launch under torchrun, one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n_gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), *sys.argv]
            raise SystemExit(subprocess.call(cmd))
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {n_gpus}")
    torch.cuda.set_device(local)
    if os.environ.get("SLIME_NO_NUMA_BIND", "0") != "1":
        # staging buffers pinned after this point live on the socket this rank's GPU hangs off
        from dlslime_b200.utils.numa import bind_to_device_numa

        bind_to_device_numa(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def max_over_ranks(value: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return value
    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_all(world: int):
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def make_inputs(T: int, rank: int, steps: int):
    """Pinned host inputs for `steps` distinct steps (seeded per rank and step)."""
    import torch

    xs, lgs = [], []
    for s in range(steps):
        g = torch.Generator().manual_seed(1000 * rank + s)
        xs.append(torch.randn((T, HIDDEN), generator=g).to(torch.bfloat16).pin_memory())
        lgs.append(torch.randn((T, E), generator=g).pin_memory())
    return xs, lgs


# ---------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    import torch

    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig

    T = T_MODE[args.mode]
    cfg = MoEConfig(num_experts=E, topk=TOPK, hidden=HIDDEN, intermediate=INTER)
    layer = ExpertParallelMoE(cfg, max_tokens=T, seed=0, fuse_dequant=args.fuse_dequant)
    tbo = None
    if args.overlap and args.mode == "normal":
        from dlslime_b200.models.moe import TwoBatchOverlapMoE

        tbo = TwoBatchOverlapMoE(cfg, max_tokens=T, weights=(layer.w_gate_up, layer.w_down))
    n_in = min(4, max(1, args.steps))
    host_x, host_lg = make_inputs(T, rank, n_in)
    dev_x = [h.cuda() for h in host_x]
    dev_lg = [h.cuda() for h in host_lg]
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x_stage = torch.empty_like(dev_x[0])
    lg_stage = torch.empty_like(dev_lg[0])

    # Decode-size steps are launch-bound: the whole layer is replayed from one CUDA graph on fixed buffers.
    graph = layer.capture(x_stage, lg_stage, out) if args.mode == "ll" and not args.no_graph else None

    fwd = tbo.forward if tbo is not None else layer.forward

    def run_layer(x, lg):
        if graph is None:
            fwd(x, lg, out=out)
        else:
            if x is not x_stage:
                x_stage.copy_(x, non_blocking=True)
                lg_stage.copy_(lg, non_blocking=True)
            graph.replay()

    def step_device(i):
        run_layer(dev_x[i % n_in], dev_lg[i % n_in])

    def step_e2e(i):
        x_stage.copy_(host_x[i % n_in], non_blocking=True)
        lg_stage.copy_(host_lg[i % n_in], non_blocking=True)
        run_layer(x_stage, lg_stage)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    # Pipelined end-to-end loop (prefill-size steps): the pinned-host -> device copy of step i+1 and the
    # device -> host copy of step i-1 run on their own streams while step i computes. Every step still copies
    # its own inputs in and its own output out, and the host consumes each result (one step late).
    class Pipelined:
        def __init__(self):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.xs = [torch.empty_like(dev_x[0]) for _ in range(2)]
            self.lgs = [torch.empty_like(dev_lg[0]) for _ in range(2)]
            self.outs = [torch.empty_like(out) for _ in range(2)]
            self.houts = [torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            self.in_ready = [torch.cuda.Event() for _ in range(2)]
            self.computed = [torch.cuda.Event() for _ in range(2)]
            self.out_done = [torch.cuda.Event() for _ in range(2)]
            self.primed = False

        def prefetch(self, i):
            b = i % 2
            with torch.cuda.stream(self.s_in):
                self.s_in.wait_event(self.computed[b])  # the previous user of this input slot has run
                self.xs[b].copy_(host_x[i % n_in], non_blocking=True)
                self.lgs[b].copy_(host_lg[i % n_in], non_blocking=True)
                self.in_ready[b].record(self.s_in)

        def __call__(self, i):
            main = torch.cuda.current_stream()
            b = i % 2
            if not self.primed:
                self.prefetch(i)
                self.primed = True
            main.wait_event(self.in_ready[b])
            main.wait_event(self.out_done[b])  # the output slot was copied out two steps ago
            fwd(self.xs[b], self.lgs[b], out=self.outs[b])
            self.computed[b].record(main)
            self.prefetch(i + 1)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.computed[b])
                self.houts[b].copy_(self.outs[b], non_blocking=True)
                self.out_done[b].record(self.s_out)
            self.out_done[1 - b].synchronize()  # the host reads the previous step's result

        def drain(self):
            self.s_in.synchronize()
            self.s_out.synchronize()
            self.primed = False

    pipe = Pipelined() if graph is None else None

    def timed(fn):
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()  # nvidia-smi needs a moment to come up: started before the warm-up, windowed below
        for i in range(args.warmup):
            fn(i)
        if fn is pipe:
            pipe.drain()
        sync_all(world)
        sampler.mark_begin()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(args.steps):
            fn(i)
        if fn is pipe:
            torch.cuda.current_stream().wait_stream(pipe.s_out)  # the last result is on the host before the clock stops
        ev1.record()
        if fn is pipe:
            pipe.drain()
        sync_all(world)
        sampler.mark_end()
        clocks = sampler.stop() if rank == 0 else None
        ms = ev0.elapsed_time(ev1) / args.steps
        layer.buf.status.check()
        if tbo is not None:
            tbo.check()
        return max_over_ranks(ms, world), clocks

    ms_dev, clocks = timed(step_device)
    ms_e2e_serial, _ = timed(step_e2e)
    ms_e2e = timed(pipe)[0] if pipe is not None else ms_e2e_serial

    # phase breakdown (one extra instrumented pass; not part of the reported value)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(7)]
    sync_all(world)
    e = None  # device-resident step counter, as in the timed loops
    # keep the GPU busy for ~1 ms first, so that the launches below are queued ahead of their execution and the short
    # phases are not measured as host launch latency
    try:
        torch.cuda._sleep(2_000_000)
    except Exception:
        torch.empty(512 << 20, dtype=torch.uint8, device="cuda").fill_(1)
    evs[0].record()
    layer.step_route(dev_lg[0], T, e)
    evs[1].record()
    layer.step_dispatch(dev_x[0], e)
    evs[2].record()
    layer.step_recv(T, e)
    evs[3].record()
    layer.step_gate_up()
    evs[4].record()
    layer.step_down()
    evs[5].record()
    layer.step_combine(out, T, e)
    evs[6].record()
    sync_all(world)
    names = ["route", "dispatch_quant_push", "recv_wait_dequant", "gate_up_swiglu_gemm", "down_gemm_combine_push", "combine_wait_reduce"]
    breakdown = {n: round(max_over_ranks(evs[i].elapsed_time(evs[i + 1]) * 1e3, world), 1) for i, n in enumerate(names)}

    weights_gb = (layer.w_gate_up.numel() + layer.w_down.numel()) * 2 / 1e9
    remote_frac = (world - 1) / world
    nvlink_bytes = T * TOPK * (HIDDEN + HIDDEN // 128 * 4 + 8) * remote_frac + T * TOPK * HIDDEN * 2 * remote_frac
    return {
        "ms_dev": ms_dev, "ms_e2e": ms_e2e, "ms_e2e_serial": ms_e2e_serial, "e2e_pipelined": pipe is not None, "clocks": clocks, "breakdown_us": breakdown, "T": T,
        "h2d": host_x[0].numel() * 2 + host_lg[0].numel() * 4, "d2h": host_out.numel() * 2,
        "launches": (18 if tbo is not None else 6) * args.steps, "cuda_graph": graph is not None, "overlap": tbo is not None,
        "dequant": "in the gate/up GEMM's A-tile loader" if args.fuse_dequant else "separate pass", "weights_gb": weights_gb, "nvlink_bytes_per_rank": nvlink_bytes,
    }


# ---------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------
def run_reference(args, rank, world, local):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dlslime")):
        return {"unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference has not been run)"}
    from baseline.reference_arm import run as run_ref_arm

    return run_ref_arm(args, rank, world, local, T_MODE[args.mode], make_inputs, sync_all, max_over_ranks, ClockSampler)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--mode", choices=["ll", "normal"], default="normal")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--fuse-dequant", action="store_true",
                    help="expand the received e4m3 rows to bf16 inside the gate/up GEMM instead of in a separate pass (measured slower)")
    ap.add_argument("--overlap", action="store_true",
                    help="normal mode: split the step into two half-batches on two streams (communication of one half under the GEMMs of the other)")
    ap.add_argument("--no-graph", action="store_true", help="ll mode: launch the kernels one by one instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    rank, world, local = init_dist(args.gpus)
    res = run_ours(args, rank, world, local) if args.impl == "ours" else run_reference(args, rank, world, local)
    if "unavailable" in res:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": res["unavailable"]}))
        return 0
    T = res["T"]
    us = res["ms_dev"] * 1e3
    line = {
        "metric": "EP dispatch+combine latency (us) [full MoE layer step: dispatch+fp8 quant -> grouped SwiGLU FFN -> combine]",
        "value": round(us, 2), "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(res["ms_dev"], 5), "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (fp8 e4m3 1x128 on the wire)", "data": "synthetic", "impl": args.impl,
        "tokens_per_s": round(world * T / (res["ms_dev"] * 1e-3), 1),
        "nvlink_gbs_per_rank": round(res["nvlink_bytes_per_rank"] / (res["ms_dev"] * 1e-3) / 1e9, 2),
        "config": {
            "model": "DeepSeek-V3-shaped MoE layer: 256 experts, top-8, hidden 7168, intermediate 2048",
            "mode": args.mode, "cuda_graph": bool(res.get("cuda_graph")), "two_batch_overlap": bool(res.get("overlap")), "dequant": res.get("dequant"), "tokens_per_rank": T, "global_batch": world * T, "seq_len": 1,
            "parallelism": f"ep{world}", "experts_per_rank": E // world,
            "l2": f"inputs larger than L2: {res['weights_gb']:.1f} GB of expert weights per rank are streamed every step",
        },
        "e2e": {"value": round(res["ms_e2e"] * 1e3, 2), "unit": "us", "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"],
                "tokens_per_s": round(world * T / (res["ms_e2e"] * 1e-3), 1),
                "copies": "overlapped with the neighbouring steps on copy streams" if res.get("e2e_pipelined") else "in line with the step",
                "serial_us": round(res.get("ms_e2e_serial", res["ms_e2e"]) * 1e3, 2)},
        "gpu_launches": res["launches"],
        "clocks": res["clocks"],
        "breakdown_us": res.get("breakdown_us"),
    }
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
