"""Real multi-GPU runs (one process per GPU over NCCL + CUDA IPC). Needs >= 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(n, *checks, timeout=600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "multigpu_worker.py"), *checks]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-4000:]
    assert res.stdout.count("WORKER_OK") == n, res.stdout[-4000:]


def test_endpoint_allgather_moe_on_all_gpus():
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    _launch(n, "endpoint", "allgather", "allgather_multicast", "alltoall", "moe", "moe_streamed", "moe_tbo", "ag_gemm", "ag_gemm_fp8", "kv", "torch_backend")
