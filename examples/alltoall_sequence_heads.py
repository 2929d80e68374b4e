#!/usr/bin/env python3
"""Sequence <-> head exchange with the low-latency all-to-all (needs 2, 4 or 8 GPUs).

    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/alltoall_sequence_heads.py

Every rank holds its slice of the sequence for ALL heads, [seq / world, heads, head_dim]; after the exchange it holds the
WHOLE sequence for its own heads, [seq, heads / world, head_dim]: the step that Ulysses-style sequence parallelism
puts in front of attention. One kernel stores every destination's rows into that rank's buffer over NVLink and publishes
a flag per source; the result is a view of the buffer. The uniform form is checked here against NCCL.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200.ops.alltoall import AllToAllLLBuffer  # noqa: E402


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    seq_local, heads, head_dim = 256, 8 * world, 128
    hpr = heads // world  # heads per rank after the exchange
    x = torch.randn(seq_local, heads, head_dim, device="cuda").to(torch.bfloat16)

    # rows for destination p = my sequence slice restricted to p's heads, one row per token
    send = x.view(seq_local, world, hpr * head_dim).transpose(0, 1).contiguous().view(world * seq_local, hpr * head_dim)
    a2a = AllToAllLLBuffer(seq_local, hpr * head_dim, torch.bfloat16)
    got = a2a.all_to_all_ll(send)  # [world * seq_local, hpr * head_dim], ordered by source rank = by sequence position
    torch.cuda.synchronize()
    a2a.status.check()
    full_seq_my_heads = got.view(world * seq_local, hpr, head_dim)

    ref = torch.empty_like(send)
    dist.all_to_all_single(ref, send)
    assert torch.equal(got, ref)
    if rank == 0:
        print(f"each rank now holds {tuple(full_seq_my_heads.shape)} = [sequence, heads / {world}, head_dim]")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
