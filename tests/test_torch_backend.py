"""The "dlslime" torch.distributed backend: send / recv / batch_isend_irecv between two CPU processes."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


import pytest


@pytest.mark.parametrize("impl", ["cpp", "python"])
def test_send_recv_between_two_processes(impl):
    """Both forms of the backend: the C++ c10d::Backend (csrc/torch/slime_backend.cpp) and the Python ProcessGroup."""
    if impl == "cpp":
        from dlslime_b200 import _build

        if _build.build_torch_plugin() is None:
            pytest.skip("the C++ backend needs an importable torch to build against")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", SLIME_TORCH_BACKEND=impl)
    port = "29641" if impl == "cpp" else "29642"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", port, os.path.join(HERE, "torch_backend_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("BACKEND_OK") == 2 and res.stdout.count(f" {impl}") >= 2
