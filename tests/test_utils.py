"""Trace merging, NVTX ranges without CUDA, and the DRAM pool's back-pressure."""
import threading
import time

import pytest

from dlslime_b200.ops.offload import DRAMMemoryPool
from dlslime_b200.utils.nvtx import nvtx_annotate, nvtx_range
from dlslime_b200.utils.profiler import dist_print, merge_traces


def test_merge_traces_remaps_pids_per_rank_and_labels_processes():
    t0 = {"traceEvents": [{"ph": "M", "name": "process_name", "pid": 7, "args": {"name": "python"}},
                          {"ph": "X", "pid": 7, "tid": 1, "name": "kernel_a", "ts": 1, "dur": 2}]}
    t1 = {"traceEvents": [{"ph": "X", "pid": 7, "tid": 1, "name": "kernel_b", "ts": 1, "dur": 2},
                          {"ph": "X", "pid": "gpu0", "tid": 3, "name": "kernel_c", "ts": 3, "dur": 1}]}
    m = merge_traces([t0, t1], names=["prefill", "decode"])
    ev = m["traceEvents"]
    by_name = {e["name"]: e for e in ev if e.get("ph") == "X"}
    assert by_name["kernel_a"]["pid"] == 7 and by_name["kernel_b"]["pid"] == 1_000_007
    assert 1_000_000 <= by_name["kernel_c"]["pid"] < 2_000_000
    labels = {e["pid"]: e["args"]["name"] for e in ev if e.get("ph") == "M" and e["name"] == "process_name"}
    assert labels[7] == "prefill: python" and labels[1_000_007] == "decode" and labels[by_name["kernel_c"]["pid"]] == "decode"
    # inputs are not modified
    assert t1["traceEvents"][0]["pid"] == 7


def test_nvtx_helpers_are_noops_without_cuda(capsys):
    calls = []

    @nvtx_annotate("labelled")
    def f(x):
        calls.append(x)
        return x + 1

    with nvtx_range("outer"):
        assert f(1) == 2
    assert calls == [1] and f.__name__ == "f"
    dist_print("hello", ranks=None)
    assert "[rank 0] hello" in capsys.readouterr().out


def test_dram_pool_blocks_when_full_and_wakes_on_release():
    pool = DRAMMemoryPool(slot_bytes=1024, num_slots=2)
    a, b = pool.acquire(), pool.acquire()
    assert {a, b} == {0, 1} and pool.slot(a).numel() == 1024
    with pytest.raises(TimeoutError):
        pool.acquire(timeout=0.05)
    got = []
    t = threading.Thread(target=lambda: got.append(pool.acquire(timeout=5)))
    t.start()
    time.sleep(0.05)
    pool.release(a)
    t.join(5)
    assert got == [a]


def test_collective_buffer_names_of_the_reference_resolve():
    import dlslime_b200 as dlslime
    from dlslime_b200.ops.allgather import AllGatherLLBuffer
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    assert dlslime.AllGatherInterLLBuffer is AllGatherLLBuffer
    assert dlslime.AllToAllIntraLLBuffer is AllToAllLLBuffer
    for name in ("buffer_info", "connect_full_mesh", "get_local_buffer", "get_buffer_size_hint", "set_max_bs", "all_to_all_ll"):
        assert callable(getattr(AllToAllLLBuffer, name))
    for name in ("buffer_info", "connect_full_mesh", "all_gather_ll", "all_gather_ll_hook"):
        assert callable(getattr(AllGatherLLBuffer, name))
    assert AllToAllLLBuffer.get_buffer_size_hint(128, 7168, __import__("torch").bfloat16, 8) == 2 * 8 * 128 * 7168 * 2 + 4096
    import pytest

    with pytest.raises(AttributeError):
        dlslime.no_such_name


def test_names_in_the_documentation_resolve():
    """Every dotted ``dlslime_b200.…`` name in the documentation and the README is importable."""
    import importlib
    import pathlib
    import re

    root = pathlib.Path(__file__).resolve().parent.parent
    files = [root / "README.md", *sorted((root / "docs").rglob("*.md"))]
    names = set()
    for f in files:
        names.update(re.findall(r"\bdlslime_b200(?:\.[A-Za-z_][A-Za-z0-9_]*)+", f.read_text()))
    assert len(names) > 10
    missing = []
    for name in sorted(names):
        parts = name.split(".")
        obj, i = None, len(parts)
        while i > 0:  # longest importable module prefix, then attributes
            try:
                obj = importlib.import_module(".".join(parts[:i]))
                break
            except ImportError:
                i -= 1
        try:
            for attr in parts[i:]:
                obj = getattr(obj, attr)
        except AttributeError:
            missing.append(name)
    assert not missing, f"documented names that do not exist: {missing}"


def test_bench_reports_unavailable_without_a_gpu():
    """On a host without CUDA both arms of bench.py print one JSON line saying so and exit 0."""
    import json
    import pathlib
    import subprocess
    import sys

    import pytest
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the benchmark itself runs under the gpu marker's tier")
    root = pathlib.Path(__file__).resolve().parent.parent
    for impl in ("ours", "reference"):
        res = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", impl, "--steps", "1", "--warmup", "3"],
                             capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stderr[-2000:]
        line = json.loads(res.stdout.strip().splitlines()[-1])
        assert line["impl"] == impl and "unavailable" in line


def test_trace_files_of_a_directory_are_merged(tmp_path):
    import gzip
    import json

    from dlslime_b200.utils import profiler

    (tmp_path / "host0").mkdir()
    (tmp_path / "host1" / "deep").mkdir(parents=True)
    ev = lambda name, pid: {"ph": "X", "name": name, "pid": pid, "tid": 1, "ts": 0, "dur": 5}
    (tmp_path / "host0" / "rank0.json").write_text(json.dumps({"traceEvents": [ev("a", 7)]}))
    with gzip.open(tmp_path / "host1" / "deep" / "rank1.json.gz", "wt") as f:
        json.dump([ev("b", 7)], f)  # bare-array form
    (tmp_path / "notes.json").write_text(json.dumps({"not": "a trace"}))
    out = tmp_path / "all.json"
    assert profiler.main(["-i", str(tmp_path), "-o", str(out)]) == 0
    merged = json.loads(out.read_text())
    xs = [e for e in merged["traceEvents"] if e["ph"] == "X"]
    assert sorted(e["name"] for e in xs) == ["a", "b"] and len({e["pid"] for e in xs}) == 2
    labels = [e["args"]["name"] for e in merged["traceEvents"] if e.get("name") == "process_name"]
    assert any("host0/rank0.json" in n for n in labels) and any("rank1.json.gz" in n for n in labels)
    import pytest

    with pytest.raises(FileNotFoundError):
        profiler.merge_trace_files(str(tmp_path / "host0" / "nothing-here"))
