"""Command-line front ends: cache CLI (parser, sizes, argv replay, runtime dir, daemon round trip) and
the native nanoctrl program (daemon round trip, obs tables)."""
import argparse
import json
import os
import subprocess
import sys
import time

import pytest

from dlslime_b200 import _build
from dlslime_b200 import _slime_c as c
from dlslime_b200.cache import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_size_parser():
    assert [cli.parse_size(s) for s in ("262144", "256K", "1G", "2GiB", "1.5M", "3 MB", "1t")] == [262144, 256 << 10, 1 << 30, 2 << 30, 1536 << 10, 3 << 20, 1 << 40]
    for bad in ("12Q", "", "1.0000001K", "-5"):
        with pytest.raises(argparse.ArgumentTypeError):
            cli.parse_size(bad)


def test_parser_defaults_argv_replay_and_mode_validation(tmp_path):
    a = cli.parse_args(["start", "--ctrl", "http://h:3000", "--memory-size", "1G"])
    assert (a.host, a.port, a.slab_size, a.memory_size, a.alias, a.metadata_only) == ("127.0.0.1", 8765, 256 << 10, 1 << 30, "cache-agent:0", False)
    replay = cli.parse_args(["__run", *cli.service_argv(a)])
    assert {k: v for k, v in vars(replay).items() if k != "command"} == {k: v for k, v in vars(a).items() if k != "command"}
    assert cli.service_mode_error(a) is None
    assert "needs --ctrl" in cli.service_mode_error(cli.parse_args(["start", "--memory-size", "1G"]))
    assert "non-zero --memory-size" in cli.service_mode_error(cli.parse_args(["start", "--ctrl", "http://h:1"]))
    assert "multiple of --slab-size" in cli.service_mode_error(cli.parse_args(["start", "--ctrl", "x", "--memory-size", "300K", "--slab-size", "128K"]))
    assert cli.service_mode_error(cli.parse_args(["start", "--metadata-only"])) is None
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps({"port": 9001, "memory-size": "2M", "scope": "s"}))
    b = cli.parse_args(["start", "--config", str(cfg), "--ctrl", "x"])
    assert (b.port, b.memory_size, b.scope) == (9001, 2 << 20, "s")


def test_runtime_dir_precedence(monkeypatch):
    monkeypatch.delenv("DLSLIME_CACHE_RUNTIME_DIR", raising=False)
    monkeypatch.delenv("XDG_RUNTIME_DIR", raising=False)
    assert str(cli.runtime_dir()) == "/tmp/dlslime-cache"
    monkeypatch.setenv("XDG_RUNTIME_DIR", "/run/user/7")
    assert str(cli.runtime_dir()) == "/run/user/7/dlslime-cache"
    monkeypatch.setenv("DLSLIME_CACHE_RUNTIME_DIR", "/x/y")
    assert str(cli.runtime_dir()) == "/x/y"


def test_cache_daemon_round_trip(tmp_path):
    env = dict(os.environ, DLSLIME_CACHE_RUNTIME_DIR=str(tmp_path), PYTHONPATH=ROOT)
    run = lambda *a: subprocess.run([sys.executable, "-m", "dlslime_b200.cache.cli", *a], env=env, capture_output=True, text=True, cwd=ROOT, timeout=60)
    assert run("status").returncode == 1
    r = run("start", "--metadata-only", "--port", "18765")
    assert r.returncode == 0 and "started" in r.stdout, r.stdout + r.stderr
    try:
        s = run("status")
        assert s.returncode == 0 and "healthy" in s.stdout
        assert "already running" in run("start", "--metadata-only", "--port", "18765").stdout
    finally:
        assert run("stop").returncode == 0
    assert run("status").returncode == 1 and not (tmp_path / "cache.json").exists()


def test_snapshot_state_and_units():
    now = 1_000_000
    assert c.ctrl.snapshot_state({"reported_at_ms": now - 1000}, now, 45000) == "alive"
    assert c.ctrl.snapshot_state({"reported_at_ms": now - 50000}, now, 45000) == "stale"
    assert c.ctrl.snapshot_state({"reported_at_ms": now, "status": "stopped"}, now, 45000) == "stopped"
    assert c.ctrl.human_bps(950) == "950 bps" and c.ctrl.human_bps(2.5e9) == "2.50 Gbps" and c.ctrl.human_bytes(3 << 20) == "3.00 MiB"


def test_nanoctrl_program_daemon_and_obs(tmp_path):
    _build.build_host()
    exe = str(_build.nanoctrl_bin_path())
    env = dict(os.environ, NANOCTRL_RUNTIME_DIR=str(tmp_path))
    run = lambda *a: subprocess.run([exe, *a], env=env, capture_output=True, text=True, timeout=60)
    r = run("start", "--host", "127.0.0.1", "--port", "13391", "--redis-port", "16391")
    assert r.returncode == 0, r.stdout + r.stderr
    try:
        assert run("status").returncode == 0
        from dlslime_b200.nanoctrl import NanoCtrlClient, RespClient

        assert NanoCtrlClient("http://127.0.0.1:13391").register_peer("1.2.3.4", alias="A")["redis_address"] == "127.0.0.1:16391"
        snap = {"schema_version": 1, "peer_id": "A", "host": "h", "pid": 1, "reported_at_ms": int(time.time() * 1000),
                "summary": {"pending_ops": 0, "completed_bytes_total": 5 << 20, "error_total": 0, "mr_count": 2}, "ewma_bandwidth_bps": 8e9,
                "nics": [{"nic": "nvlink:0", "kind": "nvlink", "pending_ops": 0, "completed_bytes_total": 5 << 20, "post_failures_total": 0,
                          "cq_errors_total": 0, "ewma_bandwidth_bps": 8e9}],
                "connections": [{"conn_id": "A->B", "peer": "B", "local_nic": "cuda:0", "remote_nic": "cuda:1", "state": "connected", "connected": True}]}
        RespClient("127.0.0.1", 16391).set("obs:peer:A", json.dumps(snap))
        peers = run("obs", "peers").stdout
        assert "A" in peers and "alive" in peers and "5.00 MiB" in peers and "8.00 Gbps" in peers
        assert "nvlink:0" in run("obs", "nics").stdout and "cuda:1" in run("obs", "links").stdout
        assert "1 alive" in run("obs", "status").stdout
        assert json.loads(run("obs", "peers", "--json").stdout)[0]["state"] == "alive"
    finally:
        assert run("stop").returncode == 0
    assert run("status").returncode == 1
