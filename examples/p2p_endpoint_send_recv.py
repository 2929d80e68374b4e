#!/usr/bin/env python3
"""The endpoint API without a control plane: two endpoints, info exchanged by hand, one-sided and two-sided I/O.

    python examples/p2p_endpoint_send_recv.py                 # TCP endpoints
    SLIME_RDMA_PROVIDER=loopback python examples/p2p_endpoint_send_recv.py --rdma   # RC queue pairs (software fabric)
    python examples/p2p_endpoint_send_recv.py --rdma          # on a host with an RDMA NIC

Covers the reference's p2p_rdma_rc_read.py, p2p_rdma_rc_write.py and p2p_rdma_rc_send_recv_*.py.
"""
import argparse
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import _slime_c  # noqa: E402


def main(use_rdma: bool):
    if use_rdma:
        a, b = _slime_c.RDMAEndpoint("", 1, "", 2), _slime_c.RDMAEndpoint("", 1, "", 2)
    else:
        a, b = _slime_c.TcpEndpoint(), _slime_c.TcpEndpoint()
    n = 1 << 20
    src = ctypes.create_string_buffer(bytes(i % 253 for i in range(n)), n)
    dst = ctypes.create_string_buffer(n)
    a.register_memory_region("src", ctypes.addressof(src), 0, n)
    b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
    ia, ib = a.endpoint_info(), b.endpoint_info()   # in a real deployment these travel through a store
    assert a.connect(ib) == 0 and b.connect(ia) == 0
    if not use_rdma:  # TCP endpoints learn remote regions explicitly
        for name, info in ib["mr_info"].items():
            a.register_remote_memory_region(name, info)
    lh, rh = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
    # assignment tuple: (local handle, remote handle, remote offset, local offset, length)
    assert a.write([(lh, rh, 0, 0, n)]).wait(10_000) == 0 and dst.raw == src.raw
    msg = ctypes.create_string_buffer(b"hello over send/recv", 32)
    got = ctypes.create_string_buffer(32)
    r = b.recv((ctypes.addressof(got), 0, 32))
    s = a.send((ctypes.addressof(msg), 0, 32))
    assert s.wait(10_000) == 0 and r.wait(10_000) == 0 and got.raw == msg.raw
    print(f"{a.kind()} endpoints: 1 MiB write and a 32-byte send/recv verified")
    a.shutdown()
    b.shutdown()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--rdma", action="store_true")
    main(ap.parse_args().rdma)
