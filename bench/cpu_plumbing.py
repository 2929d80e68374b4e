#!/usr/bin/env python
"""CPU-only plumbing check: two ranks over gloo + TCP endpoints with the control plane in-process.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29611 bench/cpu_plumbing.py

Rank 0 runs NanoCtrl inside its own process. Each rank starts a PeerAgent and registers a 64 MiB
fp32 region filled with uniform[-1, 1) values (seed 0 + rank). Rank 0 then performs 256
write + read-back operations against rank 1's region: sizes 2^k bytes with k uniform in [10, 26],
at random 64-byte-aligned offsets (seeded); every read-back is compared bit for bit with what was
written. A gloo all-gather of a [1024, 1024] fp32 N(0, 1) tensor follows and is checked bitwise
against a regeneration of every rank's tensor. Prints one JSON line with the wall time (informational).
"""
import json
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

REGION = 64 << 20
N_OPS = int(os.environ.get("SLIME_PLUMBING_OPS", "256"))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == 2, "this check is defined for exactly two ranks"
    from dlslime_b200.nanoctrl import start_local_nanoctrl
    from dlslime_b200.peer_agent import PeerAgent

    ctrl = start_local_nanoctrl() if rank == 0 else None
    box = [ctrl.url if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    agent = PeerAgent(box[0], alias=f"rank{rank}", scope="plumbing")
    g = torch.Generator().manual_seed(rank)
    region = torch.rand(REGION // 4, generator=g) * 2 - 1
    scratch = torch.zeros(REGION // 4)
    agent.register_memory_region("region", region.data_ptr(), 0, REGION)
    agent.register_memory_region("scratch", scratch.data_ptr(), 0, REGION)
    dist.barrier()
    peer = f"rank{1 - rank}"
    agent.connect_to(peer).wait(30)
    dist.barrier()
    t0 = time.perf_counter()
    moved = 0
    if rank == 0:
        rnd = np.random.default_rng(0)
        mine = region.numpy().view(np.uint8)
        back = scratch.numpy().view(np.uint8)
        for i in range(N_OPS):
            size = 1 << int(rnd.integers(10, 27))
            loff = int(rnd.integers(0, (REGION - size) // 64 + 1)) * 64
            roff = int(rnd.integers(0, (REGION - size) // 64 + 1)) * 64
            assert agent.write(peer, [("region", "region", loff, roff, size)]).wait(60) == 0
            assert agent.read(peer, [("scratch", "region", loff, roff, size)]).wait(60) == 0
            assert np.array_equal(back[loff:loff + size], mine[loff:loff + size]), f"op {i}: read-back differs"
            moved += 2 * size
    dist.barrier()
    x = torch.randn(1024, 1024, generator=torch.Generator().manual_seed(100 + rank))
    gathered = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(gathered, x)
    for r in range(world):
        ref = torch.randn(1024, 1024, generator=torch.Generator().manual_seed(100 + r))
        assert torch.equal(gathered[r].view(torch.int32), ref.view(torch.int32)), "all-gather is not bitwise equal"
    elapsed = time.perf_counter() - t0
    dist.barrier()
    agent.shutdown()
    dist.barrier()
    if rank == 0:
        ctrl.stop()
        print(json.dumps({"check": "cpu_plumbing", "ops": N_OPS, "bytes_moved": moved, "seconds": round(elapsed, 3),
                          "mb_per_s": round(moved / elapsed / 1e6, 1), "bitwise_equal": True}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
