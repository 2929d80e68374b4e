#!/usr/bin/env python3
"""SlimeRPC between two PeerAgents in one process.

    python examples/rpc_example.py                        # starts a control plane in this process
    python examples/rpc_example.py --ctrl http://host:3000  # or uses a running `nanoctrl start`

Same flow as the reference's examples/python/rpc_example.py: a service class with @method-decorated methods,
`serve` on the worker, `proxy` on the driver, futures with .wait().
"""
import argparse
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import PeerAgent  # noqa: E402
from dlslime_b200.nanoctrl import start_local_nanoctrl  # noqa: E402
from dlslime_b200.rpc import method, proxy, serve  # noqa: E402


class CalcService:
    @method
    def add(self, a: int, b: int) -> int:
        return a + b

    @method
    def mul(self, a: float, b: float) -> float:
        return a * b

    @method
    def echo(self, msg: str) -> str:
        return f"echo: {msg}"


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
        t = threading.Thread(target=serve, args=(worker, CalcService(), "driver:0"), kwargs={"stop_event": stop}, daemon=True)
        t.start()
        w = proxy(driver, "worker:0", CalcService)
        assert w.add(1, 2).wait() == 3
        assert abs(w.mul(3.14, 2.0).wait() - 6.28) < 1e-6
        assert w.echo("hello").wait() == "echo: hello"
        results = [w.add(i, i * 10).wait() for i in range(5)]
        assert results == [0, 11, 22, 33, 44]
        print(f"add / mul / echo / batch add = {results}: all calls returned")
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
