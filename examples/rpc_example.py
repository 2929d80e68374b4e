#!/usr/bin/env python3
"""SlimeRPC between two PeerAgents in one process.

    python examples/rpc_example.py                        # starts a control plane in this process
    python examples/rpc_example.py --ctrl http://host:3000  # or uses a running `nanoctrl start`

The pattern of the reference's examples/python/rpc_example.py (a class with @method-decorated methods, `serve` on the
worker, `proxy` on the driver, futures with .wait()), on a small block directory with pickled and raw methods.
"""
import argparse
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import PeerAgent  # noqa: E402
from dlslime_b200.nanoctrl import start_local_nanoctrl  # noqa: E402
from dlslime_b200.rpc import method, proxy, serve  # noqa: E402


class BlockIndex:
    """A toy block directory: which worker holds which KV block, served over SlimeRPC."""

    def __init__(self):
        self.blocks = {}

    @method
    def publish(self, block_id: int, owner: str, nbytes: int) -> int:
        self.blocks[block_id] = (owner, nbytes)
        return len(self.blocks)

    @method
    def lookup(self, block_id: int):
        return self.blocks.get(block_id)

    @method
    def total_bytes(self) -> int:
        return sum(n for _, n in self.blocks.values())

    @method(raw=True)
    def checksum(self, payload: bytes) -> bytes:
        return sum(payload).to_bytes(8, "little")


def main(ctrl_url):
    local = None
    if ctrl_url is None:
        local = start_local_nanoctrl()
        ctrl_url = local.url
    worker = PeerAgent(nanoctrl_url=ctrl_url, alias="worker:0")
    driver = PeerAgent(nanoctrl_url=ctrl_url, alias="driver:0")
    stop = threading.Event()
    try:
        driver.connect_to("worker:0").wait(10)
        worker.connect_to("driver:0").wait(10)
        print("Connected.")
        t = threading.Thread(target=serve, args=(worker, BlockIndex(), "driver:0"), kwargs={"stop_event": stop}, daemon=True)
        t.start()
        w = proxy(driver, "worker:0", BlockIndex)
        assert w.publish(7, "prefill:3", 1 << 20).wait() == 1
        futures = [w.publish(100 + i, f"prefill:{i % 4}", 4096 * (i + 1)) for i in range(8)]   # eight calls in flight
        assert [f.wait() for f in futures][-1] == 9
        assert w.lookup(7).wait() == ("prefill:3", 1 << 20) and w.lookup(999).wait() is None
        assert w.total_bytes().wait() == (1 << 20) + 4096 * 36
        assert int.from_bytes(w.checksum(bytes(range(200))).wait(), "little") == sum(range(200))
        print("publish / lookup / total_bytes / raw checksum: all calls returned")
        w.close()
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
