#!/usr/bin/env python3
"""torch.distributed send / recv on the "dlslime" backend (two ranks; CPU tensors, or CUDA tensors with --cuda).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/p2p_send_recv_torch.py [--cuda]

Counterpart of the reference's p2p_rdma_rc_send_recv_torch.py: the backend offers point-to-point operations only, which is
what pipeline stages exchange; collectives stay on NCCL or gloo in a second process group.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import dlslime_b200.torch_backend as slime_backend  # noqa: E402  (registers the backend)


def main():
    dist.init_process_group("dlslime")
    rank, peer = dist.get_rank(), 1 - dist.get_rank()
    dev = torch.device("cuda", 0) if "--cuda" in sys.argv else torch.device("cpu")
    activations = torch.full((4, 1024), float(rank + 1), device=dev)
    received = torch.empty_like(activations)
    if rank == 0:
        dist.send(activations, dst=1)
        dist.recv(received, src=1)
    else:
        dist.recv(received, src=0)
        dist.send(activations, dst=0)
    assert torch.all(received == float(peer + 1))
    # both directions at once, as a pipeline stage does between micro-batches
    out, inp = torch.arange(256.0, device=dev) + rank, torch.empty(256, device=dev)
    for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, out, peer), dist.P2POp(dist.irecv, inp, peer)]):
        work.wait()
    assert torch.equal(inp.cpu(), torch.arange(256.0) + peer)
    print(f"rank {rank}: send / recv and batch_isend_irecv verified ({slime_backend.implementation()} backend, {dev.type} tensors)", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
