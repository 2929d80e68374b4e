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
])
def test_cpu_example(script, extra, env):
    r = subprocess.run([sys.executable, os.path.join(REPO, "examples", script), *extra], env=dict(os.environ, **env),
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "verified" in r.stdout or "returned" in r.stdout
