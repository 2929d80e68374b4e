#!/usr/bin/env python
"""Headline benchmark: DeepSeek-V3-shaped expert-parallel MoE dispatch + combine.

    python bench.py --gpus N --steps K --warmup W [--mode ll|normal] [--impl ours|reference|tuned]

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
would compose them. ``--impl tuned`` is a third line for context: stock torch +
NCCL only (``all_to_all_single`` with exact splits, grouped GEMMs). Neither of
the two imports anything of this repository's package. All arms run in ONE
harness (``Harness``): the same device loop, the same serial and pipelined
end-to-end loops, a copy-only pass that shows what the host copies alone cost,
and the same correctness check against an fp32 restatement of the layer,
outside every timed region.
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
_NVML_SAMPLER = r"""
import sys, time
sel, period = sys.argv[1], float(sys.argv[2])
try:
    import pynvml as nv
    nv.nvmlInit()
    h = nv.nvmlDeviceGetHandleByUUID(sel.encode()) if sel.startswith("GPU-") else nv.nvmlDeviceGetHandleByIndex(int(sel))
    smax = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
    reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
    while True:
        t = time.time()
        sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        r = reasons(h)
        try:
            p = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:
            p = -1.0
        sys.stdout.write("%.4f,%d,%d,%.1f,%d\n" % (t, sm, smax, p, r))
        sys.stdout.flush()
        time.sleep(period)
except Exception as e:
    sys.stdout.write("error,%s\n" % (e,))
    sys.stdout.flush()
"""

# NVML clock-event reason bits (read-only queries)
_REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                0x80: "hw_power_brake_slowdown"}


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU every few milliseconds (NVML, read-only, in a child
    process so that the timed loop's thread is not disturbed); ``window(t0, t1)`` summarises the samples taken inside a
    timed region. Falls back to ``nvidia-smi -lms`` when the NVML binding is missing."""

    def __init__(self, local_index: int, period_s: float = 0.004):
        self.proc = self.path = self.out = None
        self.kind = None
        sel = str(local_index)
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if local_index < len(ids):
                sel = ids[local_index]
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen([sys.executable, "-c", _NVML_SAMPLER, sel, str(period_s)], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
            self.kind = "nvml"
        except Exception:
            self.proc = None

    def _rows(self):
        rows = []
        try:
            with open(self.path) as f:
                for line in f:
                    p = line.strip().split(",")
                    if len(p) == 5 and p[0] != "error":
                        try:
                            rows.append((float(p[0]), float(p[1]), float(p[2]), float(p[3]), int(p[4])))
                        except ValueError:
                            pass
        except OSError:
            pass
        return rows

    def window(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["clock sampler unavailable"]}
        self.out.flush()
        rows = [r for r in self._rows() if t0 <= r[0] <= t1]
        sm = sorted(r[1] for r in rows)
        reasons = set()
        for r in rows:
            for bit, name in _REASON_BITS.items():
                if r[4] & bit:
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_min_mhz": sm[0] if sm else None,
                "sm_max_mhz": max((r[2] for r in rows), default=None), "power_w_max": max((r[3] for r in rows), default=None),
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvml, 4 ms period"}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.out.close()
            try:
                os.unlink(self.path)
            except OSError:
                pass
            self.proc = None


# ---------------------------------------------------------------------------------
# distributed plumbing
# ---------------------------------------------------------------------------------
def bind_near_gpu(local: int) -> None:
    """Restrict this rank to the cores of the NUMA node its GPU hangs off (sysfs only), so that the pinned staging
    buffers allocated afterwards are local to the GPU's root port. A no-op where the platform reports no node."""
    try:
        import torch

        p = torch.cuda.get_device_properties(local)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return
        cpus = set()
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


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
        bind_near_gpu(local)  # the same for every arm; nothing of the package is imported for it
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
# one timing harness for every arm
# ---------------------------------------------------------------------------------
class Harness:
    """Times ``forward(x, logits, out)`` the same way for every arm:

    * device: inputs resident on the GPU, CUDA events around K steps;
    * end to end, serial: every step copies its inputs from pinned host memory, runs, copies its output to pinned host
      memory and synchronises;
    * end to end, pipelined (prefill-size steps): the host->device copy of step i+1 and the device->host copy of step
      i-1 run on their own streams while step i computes; every step still moves its own inputs and output, and the
      host consumes each result one step late;
    * copy floor: the pipelined loop with the step left out, i.e. what the copies alone cost on this machine with all
      ranks copying at once.
    """

    def __init__(self, forward, T, rank, world, local, args, pipelined, after=None):
        import torch

        self.torch, self.forward, self.T = torch, forward, T
        self.rank, self.world, self.local, self.args, self.after = rank, world, local, args, after
        self.n_in = min(4, max(1, args.steps))
        self.host_x, self.host_lg = make_inputs(T, rank, self.n_in)
        self.dev_x = [h.cuda() for h in self.host_x]
        self.dev_lg = [h.cuda() for h in self.host_lg]
        self.out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device="cuda")
        self.host_out = torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory()
        self.x_stage = torch.empty_like(self.dev_x[0])
        self.lg_stage = torch.empty_like(self.dev_lg[0])
        self.pipelined = pipelined
        if pipelined:
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.xs = [torch.empty_like(self.dev_x[0]) for _ in range(2)]
            self.lgs = [torch.empty_like(self.dev_lg[0]) for _ in range(2)]
            self.outs = [torch.empty_like(self.out) for _ in range(2)]
            self.houts = [torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            self.in_ready = [torch.cuda.Event() for _ in range(2)]
            self.computed = [torch.cuda.Event() for _ in range(2)]
            self.out_done = [torch.cuda.Event() for _ in range(2)]
            self.primed = False
        self.sampler = ClockSampler(local) if rank == 0 else None

    # -- step functions ---------------------------------------------------------------------------------------------
    def step_device(self, i):
        self.forward(self.dev_x[i % self.n_in], self.dev_lg[i % self.n_in], self.out)

    def step_serial(self, i, compute=True):
        torch = self.torch
        self.x_stage.copy_(self.host_x[i % self.n_in], non_blocking=True)
        self.lg_stage.copy_(self.host_lg[i % self.n_in], non_blocking=True)
        if compute:
            self.forward(self.x_stage, self.lg_stage, self.out)
        self.host_out.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    def _prefetch(self, i):
        torch, b = self.torch, i % 2
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.computed[b])  # the previous user of this input slot has run
            self.xs[b].copy_(self.host_x[i % self.n_in], non_blocking=True)
            self.lgs[b].copy_(self.host_lg[i % self.n_in], non_blocking=True)
            self.in_ready[b].record(self.s_in)

    def step_pipelined(self, i, compute=True):
        torch = self.torch
        main, b = torch.cuda.current_stream(), i % 2
        if not self.primed:
            self._prefetch(i)
            self.primed = True
        main.wait_event(self.in_ready[b])
        main.wait_event(self.out_done[b])  # the output slot was copied out two steps ago
        if compute:
            self.forward(self.xs[b], self.lgs[b], self.outs[b])
        self.computed[b].record(main)
        self._prefetch(i + 1)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.computed[b])
            self.houts[b].copy_(self.outs[b], non_blocking=True)
            self.out_done[b].record(self.s_out)
        self.out_done[1 - b].synchronize()  # the host reads the previous step's result

    def _drain(self):
        if self.pipelined:
            self.s_in.synchronize()
            self.s_out.synchronize()
            self.primed = False

    # -- timing -----------------------------------------------------------------------------------------------------
    def timed(self, fn, pipe=False, want_clocks=False):
        torch, args = self.torch, self.args
        for i in range(args.warmup):
            fn(i)
        if pipe:
            self._drain()
        sync_all(self.world)
        t0 = time.time()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(args.steps):
            fn(i)
        if pipe:
            torch.cuda.current_stream().wait_stream(self.s_out)  # the last result is on the host before the clock stops
        ev1.record()
        if pipe:
            self._drain()
        sync_all(self.world)
        t1 = time.time()
        ms = ev0.elapsed_time(ev1) / args.steps
        if self.after is not None:
            self.after()
        clocks = self.sampler.window(t0, t1) if (want_clocks and self.sampler is not None) else None
        return max_over_ranks(ms, self.world), clocks

    def run_all(self) -> dict:
        if self.sampler is not None:
            time.sleep(0.5)  # let the sampler's process come up before the first timed region
        ms_dev, clocks = self.timed(self.step_device, want_clocks=True)
        ms_serial, _ = self.timed(self.step_serial)
        copy_serial, _ = self.timed(lambda i: self.step_serial(i, compute=False))
        if self.pipelined:
            ms_e2e, _ = self.timed(self.step_pipelined, pipe=True)
            copy_floor, _ = self.timed(lambda i: self.step_pipelined(i, compute=False), pipe=True)
        else:
            ms_e2e, copy_floor = ms_serial, copy_serial
        if self.sampler is not None:
            self.sampler.stop()
        return {"ms_dev": ms_dev, "ms_e2e": ms_e2e, "ms_e2e_serial": ms_serial, "e2e_pipelined": self.pipelined,
                "copy_floor_ms": copy_floor, "copy_serial_ms": copy_serial, "clocks": clocks, "T": self.T,
                "h2d": self.host_x[0].numel() * 2 + self.host_lg[0].numel() * 4, "d2h": self.host_out.numel() * 2}

    # -- correctness, outside every timed region ----------------------------------------------------------------------
    def check(self, forward=None, n_tokens: int = 4) -> dict:
        """One step on the first input set, compared on this rank's first tokens with an fp32 restatement of the layer
        (routing, 1x128 e4m3 round trip, per-expert SwiGLU FFN with the experts' weights regenerated from their seeds,
        gate-weighted sum). Maximum over ranks."""
        torch = self.torch
        fwd = forward or self.forward
        sync_all(self.world)
        fwd(self.dev_x[0], self.dev_lg[0], self.out)
        sync_all(self.world)
        x = self.dev_x[0][:n_tokens].float()
        probs = torch.softmax(self.dev_lg[0][:n_tokens].float(), dim=-1)
        w, idx = torch.topk(probs, TOPK, dim=-1)
        xv = x.view(n_tokens, HIDDEN // 128, 128)
        scale = xv.abs().amax(-1).clamp_min(1e-4) / 448.0
        xq = (xv / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).float()
        xd = (xq * scale.unsqueeze(-1)).view(n_tokens, HIDDEN).to(torch.bfloat16).float()
        ref = torch.zeros((n_tokens, HIDDEN), dtype=torch.float32, device="cuda")
        gen = torch.Generator(device="cuda")
        for e in sorted(set(idx.flatten().tolist())):
            gen.manual_seed(e)  # seed 0 of the layer: expert e is drawn from generator seed 0 * 100003 + e
            w13 = torch.randn((2 * INTER, HIDDEN), generator=gen, device="cuda").mul_(0.02).to(torch.bfloat16).float()
            w2 = torch.randn((HIDDEN, INTER), generator=gen, device="cuda").mul_(0.02).to(torch.bfloat16).float()
            sel = (idx == e)
            tok = sel.any(-1).nonzero().flatten()
            gu = xd[tok] @ w13.t()
            h = (torch.nn.functional.silu(gu[:, :INTER]) * gu[:, INTER:]).to(torch.bfloat16).float()
            y = (h @ w2.t()).to(torch.bfloat16).float()
            ref[tok] += (w[tok] * sel[tok]).sum(-1, keepdim=True) * y
        got = self.out[:n_tokens].float()
        err = (got - ref).abs().max().item()
        mag = ref.abs().mean().item()
        err, rel = max_over_ranks(err, self.world), max_over_ranks(err / max(mag, 1e-12), self.world)
        return {"checked": True, "tokens_per_rank_checked": n_tokens, "max_err": round(err, 6),
                "max_err_over_mean_abs": round(rel, 4), "ok": bool(rel < 0.15)}


# ---------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------
def run_ours(args, rank, world, local):
    import torch

    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig

    T = T_MODE[args.mode]
    cfg = MoEConfig(num_experts=E, topk=TOPK, hidden=HIDDEN, intermediate=INTER)
    layer = ExpertParallelMoE(cfg, max_tokens=T, seed=0, fuse_dequant=args.fuse_dequant, streamed=args.phases == "streamed" and args.mode == "normal")
    tbo = None
    if args.overlap and args.mode == "normal":
        from dlslime_b200.models.moe import TwoBatchOverlapMoE

        tbo = TwoBatchOverlapMoE(cfg, max_tokens=T, weights=(layer.w_gate_up, layer.w_down))
    fwd = tbo.forward if tbo is not None else layer.forward

    def after():
        layer.buf.status.check()
        if tbo is not None:
            tbo.check()

    h = Harness(None, T, rank, world, local, args, pipelined=args.mode == "normal", after=after)
    # Decode-size steps are launch-bound: the whole layer is replayed from one CUDA graph on fixed buffers.
    graph = layer.capture(h.x_stage, h.lg_stage, h.out) if args.mode == "ll" and not args.no_graph else None

    def forward(x, lg, out):
        if graph is None:
            fwd(x, lg, out=out)
            return
        if x is not h.x_stage:
            h.x_stage.copy_(x, non_blocking=True)
            h.lg_stage.copy_(lg, non_blocking=True)
        graph.replay()  # writes h.out, the buffer every caller of the harness passes
        if out is not h.out:
            out.copy_(h.out, non_blocking=True)

    h.forward = forward
    tuned = None
    if args.phases == "auto" and args.mode == "normal" and tbo is None and not args.fuse_dequant:
        tuned = layer.autotune(h.dev_x[0], h.dev_lg[0], h.out)  # the layer's own choice, made outside every timed region
    res = h.run_all()
    res["check"] = h.check()

    # phase breakdown (one extra instrumented pass; not part of the reported value)
    dev_x, dev_lg, out = h.dev_x, h.dev_lg, h.out
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
    after()

    res.update({
        "breakdown_us": dict(breakdown, note="one extra pass with the phases run one after the other, whatever the timed loop does"),
        "launches": (18 if tbo is not None else 8 if layer.streamed else 6) * args.steps, "cuda_graph": graph is not None, "overlap": tbo is not None,
        "weights_gb": (layer.w_gate_up.numel() + layer.w_down.numel()) * 2 / 1e9,
        "notes": {"dequant": "in the gate/up GEMM's A-tile loader" if args.fuse_dequant else "separate pass",
                  "phases": "dispatch, receive and gate/up GEMM at the same time (per-expert arrival words)" if layer.streamed else "one after the other",
                  "expert_gemm": {False: "single CTAs, 128 x 256 tiles", True: "CTA pairs, 256 x 256 tiles", "wide": "CTA pairs, 256 x 512 tiles", "swap": "CTA pairs, operands swapped: 256 weight rows x up to 256 tokens"}[layer.pair_gemm],
                  "phases_autotune": tuned,
                  "transport": "in-kernel stores and bulk copies to NVLink peer memory"},
    })
    return res


# ---------------------------------------------------------------------------------
# baseline arms
# ---------------------------------------------------------------------------------
def run_reference(args, rank, world, local):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "dlslime")):
        return {"unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref of the reference has not been run)"}
    from baseline.reference_arm import run as run_ref_arm

    return run_ref_arm(args, rank, world, local, T_MODE[args.mode], Harness)


def run_tuned(args, rank, world, local):
    from baseline.tuned_arm import run as run_tuned_arm

    return run_tuned_arm(args, rank, world, local, T_MODE[args.mode], Harness)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--mode", choices=["ll", "normal"], default="normal")
    ap.add_argument("--impl", choices=["ours", "reference", "tuned"], default="ours",
                    help="ours: this repository; reference: the unmodified reference package + torch/NCCL; tuned: stock torch + NCCL, well used")
    ap.add_argument("--fuse-dequant", action="store_true",
                    help="expand the received e4m3 rows to bf16 inside the gate/up GEMM instead of in a separate pass (measured slower)")
    ap.add_argument("--overlap", action="store_true",
                    help="normal mode: split the step into two half-batches on two streams (communication of one half under the GEMMs of the other)")
    ap.add_argument("--phases", choices=["auto", "serial", "streamed"], default="auto",
                    help="dispatch, receive and the gate/up GEMM one after the other (serial), at the same time (streamed), or "
                         "whichever the layer measures as faster for this shape before the timed region (auto; prefill mode only)")
    ap.add_argument("--no-graph", action="store_true", help="ll mode: launch the kernels one by one instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    rank, world, local = init_dist(args.gpus)
    res = {"ours": run_ours, "reference": run_reference, "tuned": run_tuned}[args.impl](args, rank, world, local)
    if "unavailable" in res:
        if rank == 0:
            print(json.dumps({"impl": args.impl, "unavailable": res["unavailable"]}))
        return 0
    T = res["T"]
    us = res["ms_dev"] * 1e3
    remote_frac = (world - 1) / world
    nvlink_bytes = T * TOPK * (HIDDEN + HIDDEN // 128 * 4 + 8) * remote_frac + T * TOPK * HIDDEN * 2 * remote_frac
    pipelined = bool(res.get("e2e_pipelined"))
    line = {
        "metric": "EP dispatch+combine latency (us) [full MoE layer step: dispatch+fp8 quant -> grouped SwiGLU FFN -> combine]",
        "value": round(us, 2), "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(res["ms_dev"], 5), "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (fp8 e4m3 1x128 on the wire)", "data": "synthetic", "impl": args.impl,
        "tokens_per_s": round(world * T / (res["ms_dev"] * 1e-3), 1),
        "nvlink_gbs_per_rank": round(nvlink_bytes / (res["ms_dev"] * 1e-3) / 1e9, 2),
        # the workload only: identical for every arm
        "config": {
            "model": "DeepSeek-V3-shaped MoE layer: 256 experts, top-8, hidden 7168, intermediate 2048",
            "mode": args.mode, "tokens_per_rank": T, "global_batch": world * T, "seq_len": 1,
            "parallelism": f"ep{world}", "experts_per_rank": E // world,
            "l2": f"inputs larger than L2: {res['weights_gb']:.1f} GB of expert weights per rank are streamed every step",
        },
        # one harness for every arm: the same loops, the same copies, the same synchronisation points
        "e2e": {"value": round(res["ms_e2e"] * 1e3, 2), "unit": "us", "h2d_bytes_per_step": res["h2d"],
                "d2h_bytes_per_step": res["d2h"],
                "tokens_per_s": round(world * T / (res["ms_e2e"] * 1e-3), 1),
                "copies": "overlapped with the neighbouring steps on copy streams" if pipelined else "in line with the step",
                "serial_us": round(res["ms_e2e_serial"] * 1e3, 2),
                "copy_only_us": round(res["copy_floor_ms"] * 1e3, 2),
                "copy_only_serial_us": round(res["copy_serial_ms"] * 1e3, 2)},
        "gpu_launches": res["launches"],
        "clocks": res["clocks"],
        "check": res.get("check"),
        "impl_details": dict(res.get("notes") or {}, cuda_graph=bool(res.get("cuda_graph")), two_batch_overlap=bool(res.get("overlap"))),
        "breakdown_us": res.get("breakdown_us"),
    }
    if "reference_package_used" in res:
        line["reference_package_used"] = res["reference_package_used"]
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
