"""The "dlslime" torch.distributed backend: send / recv / batch_isend_irecv between two CPU processes."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_send_recv_between_two_processes():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(HERE, "torch_backend_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("BACKEND_OK") == 2
