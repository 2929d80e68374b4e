#!/usr/bin/env python3
"""Named one-sided I/O between two PeerAgents found through the control plane.

    python examples/p2p_ctrl_plane.py                     # TCP links, control plane started in this process
    SLIME_RDMA_PROVIDER=loopback python examples/p2p_ctrl_plane.py --link RoCE --devices rdma_lo0 rdma_lo2
    python examples/p2p_ctrl_plane.py --ctrl http://host:3000 --link RoCE      # real NICs

Covers what the reference's p2p_rdma_rc_read_ctrl_plane.py / p2p_rdma_rc_write_with_imm_data.py /
p2p_rdma_multi_agents_ctrl_plane.py show: register regions by name, connect_to(alias), write / read with
(region, local_off, remote_off, len) tuples, write_with_imm + imm_recv.
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
    dev_a, dev_b = (args.devices + [None, None])[:2]
    a = PeerAgent(ctrl, alias="initiator", device=dev_a, link_type=args.link)
    b = PeerAgent(ctrl, alias="target", device=dev_b, link_type=args.link)
    try:
        n = 1 << 20
        src = ctypes.create_string_buffer(bytes(i % 251 for i in range(n)), n)
        dst = ctypes.create_string_buffer(n)
        a.register_memory_region("kv", ctypes.addressof(src), 0, n)
        b.register_memory_region("kv", ctypes.addressof(dst), 0, n)
        conn = a.connect_to("target", local_device=dev_a, peer_device=dev_b).wait(10)
        print("connected:", conn.conn_id)
        assert a.write("target", [("kv", 0, 4096, 65536)]).wait(10) == 0
        assert dst.raw[4096:4096 + 65536] == src.raw[:65536]
        back = ctypes.create_string_buffer(65536)
        a.register_memory_region("back", ctypes.addressof(back), 0, 65536)
        assert a.read("target", ("back", "kv", 0, 4096, 65536)).wait(10) == 0 and back.raw == src.raw[:65536]
        assert a.write_with_imm("target", [("kv", 0, 0, 64)], imm_data=1234).wait(10) == 0
        b.query_connection("initiator").wait(5)
        ev = b.imm_recv("initiator")
        assert ev.wait(10) == 0 and ev.imm_data() == 1234
        print("write, read and write_with_imm(1234) verified")
    finally:
        a.shutdown()
        b.shutdown()
        if local is not None:
            local.stop()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctrl", default=None)
    ap.add_argument("--link", default=None, help="TCP | RoCE | IB | NVLink (default: what the host offers)")
    ap.add_argument("--devices", nargs="*", default=[], help="device of the initiator and of the target")
    main(ap.parse_args())
