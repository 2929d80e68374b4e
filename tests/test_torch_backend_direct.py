"""The GPU-direct send / recv protocol of the "dlslime" backend (dlslime_b200/torch_direct.py) on two CPU ranks, with
shared memory standing in for CUDA IPC (SLIME_BACKEND_DIRECT=shm): ordering, exchange patterns, many operations in
flight, size mismatch. The CUDA form runs in the GPU tests."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("impl", ["cpp", "python"])
def test_rendezvous_protocol_over_shared_memory(impl):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", SLIME_TORCH_BACKEND=impl, SLIME_BACKEND_DIRECT="shm")
    port = "29661" if impl == "cpp" else "29662"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", port, os.path.join(HERE, "torch_direct_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("DIRECT_OK") == 2
