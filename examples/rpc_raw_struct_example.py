#!/usr/bin/env python3
"""SlimeRPC with a hand-packed binary message instead of pickle: a raw method whose request and reply are structs.

    python examples/rpc_raw_struct_example.py [--ctrl http://host:3000]

The role of the reference's rpc_flatbuf_example.py (a schema-defined binary payload on a raw method); the layout here is
a fixed little-endian header plus a float32 vector, packed with `struct` / `numpy`, so nothing is pickled on either side:
request  = u32 op | u32 count | f32[count]        reply = u32 count | f64 sum | f32 min | f32 max
"""
import argparse
import os
import struct
import sys
import threading

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import PeerAgent  # noqa: E402
from dlslime_b200.nanoctrl import start_local_nanoctrl  # noqa: E402
from dlslime_b200.rpc import method, proxy, serve  # noqa: E402

OP_STATS = 1


class VectorService:
    @method(raw=True)
    def call(self, payload: bytes) -> bytes:
        op, count = struct.unpack_from("<II", payload, 0)
        values = np.frombuffer(payload, dtype="<f4", count=count, offset=8)
        if op != OP_STATS:
            raise ValueError(f"unknown op {op}")
        return struct.pack("<Idff", count, float(values.astype(np.float64).sum()), float(values.min()), float(values.max()))


def main(ctrl_url):
    local = None
    if ctrl_url is None:
        local = start_local_nanoctrl()
        ctrl_url = local.url
    worker = PeerAgent(nanoctrl_url=ctrl_url, alias="vec-worker:0")
    driver = PeerAgent(nanoctrl_url=ctrl_url, alias="vec-driver:0")
    stop = threading.Event()
    try:
        driver.connect_to("vec-worker:0").wait(10)
        worker.connect_to("vec-driver:0").wait(10)
        threading.Thread(target=serve, args=(worker, VectorService(), "vec-driver:0"), kwargs={"stop_event": stop}, daemon=True).start()
        svc = proxy(driver, "vec-worker:0", VectorService)
        values = np.linspace(-3.0, 5.0, 10_000, dtype="<f4")
        reply = svc.call(struct.pack("<II", OP_STATS, values.size) + values.tobytes()).wait(10)
        count, total, lo, hi = struct.unpack("<Idff", reply)
        assert count == values.size and abs(total - float(values.astype(np.float64).sum())) < 1e-6 and (lo, hi) == (-3.0, 5.0)
        try:
            svc.call(struct.pack("<II", 99, 0)).wait(10)
            raise SystemExit("the unknown op should have raised on the server")
        except Exception as e:  # the remote ValueError arrives as RemoteRpcError
            assert "unknown op 99" in str(e)
        print(f"raw struct call: {count} floats, sum {total:.3f}, remote error reported: all calls returned")
        svc.close()
    finally:
        stop.set()
        driver.shutdown()
        worker.shutdown()
        if local is not None:
            local.stop()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctrl", default=None)
    main(ap.parse_args().ctrl)
