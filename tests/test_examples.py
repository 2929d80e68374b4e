"""The CPU examples run to completion as a user would run them."""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,extra,env", [
    ("p2p_endpoint_send_recv.py", [], {}),
    ("p2p_endpoint_send_recv.py", ["--rdma"], {"SLIME_RDMA_PROVIDER": "loopback"}),
    ("p2p_ctrl_plane.py", [], {}),
    ("p2p_ctrl_plane.py", ["--link", "RoCE", "--devices", "rdma_lo0", "rdma_lo2"], {"SLIME_RDMA_PROVIDER": "loopback"}),
    ("rpc_example.py", [], {}),
    ("cache_client_example.py", [], {}),
    ("p2p_multi_agents_ctrl_plane.py", ["--workers", "4"], {}),
    ("rpc_raw_struct_example.py", [], {}),
])
def test_cpu_example(script, extra, env):
    r = subprocess.run([sys.executable, os.path.join(REPO, "examples", script), *extra], env=dict(os.environ, **env),
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "verified" in r.stdout or "returned" in r.stdout


def test_torch_send_recv_example():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29672", os.path.join(REPO, "examples", "p2p_send_recv_torch.py")]
    r = subprocess.run(cmd, env=dict(os.environ, MASTER_ADDR="127.0.0.1"), capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("verified") == 2
