"""Two processes over gloo + TCP endpoints + in-process NanoCtrl: bitwise plumbing check."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_cpu_plumbing_is_bitwise_exact():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", SLIME_PLUMBING_OPS="48")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(ROOT, "bench", "cpu_plumbing.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["bitwise_equal"] and out["ops"] == 48 and out["bytes_moved"] > 0
