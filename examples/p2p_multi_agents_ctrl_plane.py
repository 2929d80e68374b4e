#!/usr/bin/env python3
"""Several PeerAgents around one store of blocks: three workers push their block to a collector and read a peer's back.

    python examples/p2p_multi_agents_ctrl_plane.py [--workers 3] [--ctrl http://host:3000]

The shape of the reference's p2p_rdma_multi_agents_ctrl_plane.py: every agent registers under its own alias, lists the
others through the control plane, connects to the ones it needs and moves bytes by region name. Here the collector
owns one region with a slot per worker; worker i writes slot i and then reads slot (i + 1) % n, which its neighbour wrote.
"""
import argparse
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import PeerAgent  # noqa: E402
from dlslime_b200.nanoctrl import start_local_nanoctrl  # noqa: E402


def main(args):
    local = None if args.ctrl else start_local_nanoctrl()
    ctrl = args.ctrl or local.url
    n, slot = args.workers, 64 << 10
    agents = []
    try:
        collector = PeerAgent(ctrl, alias="collector", scope="example-multi")
        agents.append(collector)
        store = ctypes.create_string_buffer(n * slot)
        collector.register_memory_region("store", ctypes.addressof(store), 0, n * slot)
        workers, blocks, backs = [], [], []
        for i in range(n):
            w = PeerAgent(ctrl, alias=f"worker:{i}", scope="example-multi")
            agents.append(w)
            blk = ctypes.create_string_buffer(bytes((i * 37 + j) % 256 for j in range(slot)), slot)
            back = ctypes.create_string_buffer(slot)
            w.register_memory_region("block", ctypes.addressof(blk), 0, slot)
            w.register_memory_region("back", ctypes.addressof(back), 0, slot)
            workers.append(w), blocks.append(blk), backs.append(back)
        assert sorted(collector.list_agents()) == sorted(["collector"] + [f"worker:{i}" for i in range(n)])
        for w in workers:
            w.connect_to("collector").wait(10)
        for i, w in enumerate(workers):  # every worker writes its slot ...
            assert w.write("collector", [("block", "store", 0, i * slot, slot)]).wait(10) == 0
        for i, w in enumerate(workers):  # ... and reads the slot of its neighbour
            j = (i + 1) % n
            assert w.read("collector", [("back", "store", 0, j * slot, slot)]).wait(10) == 0
            assert backs[i].raw == blocks[j].raw
        assert store.raw == b"".join(b.raw for b in blocks)
        print(f"{n} workers wrote {n * slot >> 10} KiB into the collector and read their neighbours' blocks back: verified")
    finally:
        for a in reversed(agents):
            a.shutdown()
        if local is not None:
            local.stop()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctrl", default=None)
    ap.add_argument("--workers", type=int, default=3)
    main(ap.parse_args())
