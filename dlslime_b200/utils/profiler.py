"""Timing and trace helpers for multi-rank jobs.

* ``perf_func``     CUDA-event timing of a callable (warm-up, iterations, optional L2 flush).
* ``group_profile`` context manager: torch.profiler on every rank, per-rank Chrome traces, gathered to
                    rank 0 and merged into one timeline with one process row per rank (pid / tid remapped).
* ``merge_traces``  the merging step on its own, for traces collected elsewhere.
* ``dist_print``    print from selected ranks with a rank prefix.
* ``make_tensor``   seeded synthetic tensors for benchmarks.

Same tool set as the reference's ``dlslime/utils/json_merger.py`` (``:48-132,366-434`` in the reference), written
against plain torch.
"""

from __future__ import annotations

import contextlib
import gzip
import json
import os
import tempfile
from typing import Callable, Iterable

import torch
import torch.distributed as dist


def dist_print(*args, ranks: Iterable[int] | None = (0,), prefix: bool = True, **kw) -> None:
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if ranks is None or rank in ranks:
        print(*((f"[rank {rank}]",) if prefix else ()), *args, **kw, flush=True)


def make_tensor(shape, dtype=torch.bfloat16, device="cuda", seed: int = 0, scale: float = 1.0, kind: str = "normal") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    if kind == "normal":
        t = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * scale
    elif kind == "uniform":
        t = (torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 2 - 1) * scale
    else:
        raise ValueError(f"unknown kind {kind!r}")
    return t.to(dtype)


_flush_buf = None


def perf_func(fn: Callable[[], object], iters: int = 20, warmup: int = 3, flush_l2: bool = False):
    """Returns (last result, mean milliseconds per call) measured with CUDA events on the current stream."""
    global _flush_buf
    out = None
    for _ in range(warmup):
        out = fn()
    torch.cuda.synchronize()
    if flush_l2:
        if _flush_buf is None:
            _flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        total = 0.0
        for _ in range(iters):
            _flush_buf.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return out, total / iters
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        out = fn()
    e1.record()
    torch.cuda.synchronize()
    return out, e0.elapsed_time(e1) / iters


def merge_traces(traces: list[dict], names: list[str] | None = None) -> dict:
    """Merge Chrome traces (one per rank) into one: rank r's processes become pid ``r * 1_000_000 + pid``."""
    merged = {"traceEvents": [], "displayTimeUnit": "ms"}
    for r, tr in enumerate(traces):
        label = names[r] if names else f"rank {r}"
        seen = set()
        for ev in tr.get("traceEvents", []):
            ev = dict(ev)
            pid = ev.get("pid", 0)
            new_pid = r * 1_000_000 + (pid if isinstance(pid, int) else abs(hash(pid)) % 1_000_000)
            ev["pid"] = new_pid
            if ev.get("ph") == "M" and ev.get("name") == "process_name":
                ev["args"] = {"name": f"{label}: {ev.get('args', {}).get('name', '')}"}
                seen.add(new_pid)
            merged["traceEvents"].append(ev)
        for pid in {e["pid"] for e in merged["traceEvents"] if e["pid"] // 1_000_000 == r} - seen:
            merged["traceEvents"].append({"ph": "M", "name": "process_name", "pid": pid, "args": {"name": label}})
            merged["traceEvents"].append({"ph": "M", "name": "process_sort_index", "pid": pid, "args": {"sort_index": pid}})
    return merged


@contextlib.contextmanager
def group_profile(name: str = "trace", out_dir: str = "prof", enabled: bool = True, group=None, with_stack: bool = False):
    """Profile the enclosed region on every rank and leave ``{out_dir}/{name}.merged.json.gz`` on rank 0."""
    if not enabled:
        yield None
        return
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    prof = torch.profiler.profile(activities=acts, with_stack=with_stack)
    prof.start()
    try:
        yield prof
    finally:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        prof.stop()
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "t.json")
            prof.export_chrome_trace(path)
            with open(path) as f:
                mine = json.load(f)
        distributed = dist.is_available() and dist.is_initialized()
        rank = dist.get_rank(group) if distributed else 0
        world = dist.get_world_size(group) if distributed else 1
        gathered = [None] * world
        if distributed and world > 1:
            dist.gather_object(mine, gathered if rank == 0 else None, dst=0, group=group)
        else:
            gathered = [mine]
        if rank == 0:
            os.makedirs(out_dir, exist_ok=True)
            with gzip.open(os.path.join(out_dir, f"{name}.merged.json.gz"), "wt") as f:
                json.dump(merge_traces(gathered), f)


def merge_trace_files(input_dir: str, output: str | None = None) -> str:
    """Merge every Chrome trace (``*.json`` / ``*.json.gz``) found under ``input_dir`` (recursively, in sorted order) into
    one file; the rank label of a trace is its path relative to ``input_dir``. Returns the output path. The job of the
    reference's ``dlslime/utils/json_merge_manually.py``: traces written per rank by separate runs or hosts, merged later."""
    import pathlib
    import time

    root = pathlib.Path(input_dir)
    files = sorted(p for p in root.rglob("*") if p.is_file() and (p.name.endswith(".json") or p.name.endswith(".json.gz"))
                   and ".merged." not in p.name)
    if not files:
        raise FileNotFoundError(f"no trace files under {input_dir}")
    traces, names = [], []
    for p in files:
        opener = gzip.open if p.name.endswith(".gz") else open
        with opener(p, "rt") as f:
            data = json.load(f)
        if isinstance(data, list):  # the bare-array form of the trace format
            data = {"traceEvents": data}
        if "traceEvents" not in data:
            continue
        traces.append(data)
        names.append(str(p.relative_to(root)))
    if not traces:
        raise ValueError(f"none of the {len(files)} JSON files under {input_dir} is a Chrome trace")
    out = output or str(root / f"merged_trace_{time.strftime('%Y%m%d_%H%M%S')}.merged.json.gz")
    opener = gzip.open if out.endswith(".gz") else open
    with opener(out, "wt") as f:
        json.dump(merge_traces(traces, names), f)
    return out


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="python -m dlslime_b200.utils.profiler",
                                 description="Merge the Chrome traces found under a directory into one trace, one process group per file.")
    ap.add_argument("-i", "--input-dir", required=True)
    ap.add_argument("-o", "--output", default=None, help="output file (.json or .json.gz); default: merged_trace_<time>.merged.json.gz in the input directory")
    a = ap.parse_args(argv)
    print(merge_trace_files(a.input_dir, a.output))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
