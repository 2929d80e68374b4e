"""The "dlslime" torch.distributed backend with CUDA tensors (two processes on one GPU, staged through host memory)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("impl", ["cpp", "python"])
def test_cuda_tensors_between_two_processes(impl):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", SLIME_TORCH_BACKEND=impl)
    port = "29651" if impl == "cpp" else "29652"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", port, os.path.join(HERE, "torch_backend_worker.py"), "--cuda"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("BACKEND_OK") == 2 and res.stdout.count(f" {impl}") >= 2
