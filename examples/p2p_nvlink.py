#!/usr/bin/env python3
"""Batched scatter / gather between two GPUs through the kernel-driven NVLink endpoint (needs 2 GPUs).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/p2p_nvlink.py

Counterpart of the reference's examples/python/p2p_nvlink.py; here one kernel moves the whole batch (read AND
write), where the reference issues one cudaMemcpyAsync per assignment and supports read only.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200.ops.nvlink import NVLinkEndpoint  # noqa: E402


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peer = rank ^ 1
    seg, n = 64 << 10, 256
    buf = torch.full((2 * n * seg,), rank + 1, dtype=torch.uint8, device="cuda")
    ep = NVLinkEndpoint()
    ep.register_memory_region(buf.data_ptr(), 0, buf.numel(), "buf")
    infos = [None] * dist.get_world_size()
    dist.all_gather_object(infos, ep.endpoint_info())
    ep.connect(infos[peer])
    dist.barrier()
    if rank == 0:
        # gather n scattered 64 KiB segments of the peer's upper half into my lower half, in one launch
        perm = torch.randperm(n).tolist()
        ep.read([("buf", "buf", (n + p) * seg, i * seg, seg) for i, p in enumerate(perm)]).wait()
        assert bool((buf[: n * seg] == 2).all())
        # and scatter my upper half into the peer's lower half
        ep.write([("buf", "buf", p * seg, (n + i) * seg, seg) for i, p in enumerate(perm)]).wait()
        print(f"moved {2 * n * seg >> 20} MiB in two kernel launches")
    dist.barrier()
    if rank == 1:
        torch.cuda.synchronize()
        assert bool((buf[: n * seg] == 1).all())
    ep.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
