#!/usr/bin/env python
"""Host-side benchmarks of the endpoint API and the services on top of it (no GPU needed).

    python bench/host_bench.py io        [--transport tcp|rdma] [--sizes 4096,65536,1048576,16777216] [--batch 1] [--concurrency 1] [--iters 200]
    python bench/host_bench.py sendrecv  [--transport tcp|rdma] [--sizes ...]
    python bench/host_bench.py rpc       [--sizes 64,4096,65536,1048576] [--iters 500]
    python bench/host_bench.py cache     [--length 16777216] [--iters 20]
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 bench/host_bench.py torch [--sizes ...]
                                         # send / recv through torch.distributed with backend "dlslime"

`--transport rdma` uses the verbs provider the host offers; `SLIME_RDMA_PROVIDER=loopback` selects the software RC
fabric (which measures the engine's own overhead: striping, credits, completion routing, not a wire). One JSON line per
measurement. Counterparts in the reference: bench/python/endpoint_io_bench.py, endpoint_sendrecv_bench.py,
rpc_bench_slime_*.py and cache_bench.py (in the reference).
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import _slime_c  # noqa: E402


def make_pair(transport: str, qp: int):
    if transport == "rdma":
        a, b = _slime_c.RDMAEndpoint("", 1, "", qp), _slime_c.RDMAEndpoint("", 1, "", qp)
    else:
        a, b = _slime_c.TcpEndpoint("127.0.0.1", 0, qp), _slime_c.TcpEndpoint("127.0.0.1", 0, qp)
    return a, b


def link(a, b, transport):
    ia, ib = a.endpoint_info(), b.endpoint_info()
    assert a.connect(ib) == 0 and b.connect(ia) == 0
    if transport != "rdma":
        for name, info in ib["mr_info"].items():
            a.register_remote_memory_region(name, info)
        for name, info in ia["mr_info"].items():
            b.register_remote_memory_region(name, info)


def pct(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(len(xs) * p))]


def cmd_io(args):
    sizes = [int(s) for s in args.sizes.split(",")]
    cap = max(sizes) * args.batch
    src, dst = ctypes.create_string_buffer(cap), ctypes.create_string_buffer(cap)
    a, b = make_pair(args.transport, args.qp)
    a.register_memory_region("src", ctypes.addressof(src), 0, cap)
    b.register_memory_region("dst", ctypes.addressof(dst), 0, cap)
    link(a, b, args.transport)
    lh, rh = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
    for op in ("write", "read"):
        for size in sizes:
            batch = [(lh, rh, i * size, i * size, size) for i in range(args.batch)]
            fn = getattr(a, op)
            for _ in range(5):
                fn(batch).wait(30000)
            lat = []
            t0 = time.perf_counter()
            for _ in range(args.iters):
                t = time.perf_counter()
                futs = [fn(batch) for _ in range(args.concurrency)]  # `concurrency` operations of `batch` pieces in flight
                for f in futs:
                    f.wait(30000)
                lat.append(time.perf_counter() - t)
            dt = time.perf_counter() - t0
            print(json.dumps({"bench": "endpoint_io", "transport": a.kind(), "op": op, "bytes": size, "batch": args.batch,
                              "concurrency": args.concurrency, "qp": args.qp,
                              "p50_us": round(pct(lat, 0.5) * 1e6, 1), "p99_us": round(pct(lat, 0.99) * 1e6, 1),
                              "mb_s": round(size * args.batch * args.concurrency * args.iters / dt / 1e6, 1)}), flush=True)
    a.shutdown()
    b.shutdown()


def cmd_sendrecv(args):
    sizes = [int(s) for s in args.sizes.split(",")]
    cap = max(sizes)
    src, dst = ctypes.create_string_buffer(cap), ctypes.create_string_buffer(cap)
    a, b = make_pair(args.transport, args.qp)
    link(a, b, args.transport)
    for size in sizes:
        lat = []
        t0 = time.perf_counter()
        for _ in range(args.iters):
            t = time.perf_counter()
            r = b.recv((ctypes.addressof(dst), 0, size))
            s = a.send((ctypes.addressof(src), 0, size))
            assert s.wait(30000) == 0 and r.wait(30000) == 0
            lat.append(time.perf_counter() - t)
        dt = time.perf_counter() - t0
        print(json.dumps({"bench": "endpoint_sendrecv", "transport": a.kind(), "bytes": size, "qp": args.qp,
                          "p50_us": round(pct(lat, 0.5) * 1e6, 1), "p99_us": round(pct(lat, 0.99) * 1e6, 1),
                          "mb_s": round(size * args.iters / dt / 1e6, 1)}), flush=True)
    a.shutdown()
    b.shutdown()


def cmd_rpc(args):
    from dlslime_b200 import PeerAgent
    from dlslime_b200.nanoctrl import start_local_nanoctrl
    from dlslime_b200.rpc import method, proxy, serve

    class Echo:
        @method(raw=True)
        def echo(self, payload: bytes) -> bytes:
            return payload

    ctrl = start_local_nanoctrl()
    w, d = PeerAgent(ctrl.url, alias="worker"), PeerAgent(ctrl.url, alias="driver")
    stop = threading.Event()
    try:
        d.connect_to("worker").wait(10)
        w.connect_to("driver").wait(10)
        threading.Thread(target=serve, args=(w, Echo(), "driver"), kwargs={"stop_event": stop}, daemon=True).start()
        p = proxy(d, "worker", Echo)
        for size in [int(s) for s in args.sizes.split(",")]:
            payload = bytes(size)
            for _ in range(20):
                p.echo(payload).wait()
            lat = []
            for _ in range(args.iters):
                t = time.perf_counter()
                p.echo(payload).wait()
                lat.append(time.perf_counter() - t)
            print(json.dumps({"bench": "slimerpc_echo", "bytes": size, "p50_us": round(pct(lat, 0.5) * 1e6, 1),
                              "p99_us": round(pct(lat, 0.99) * 1e6, 1), "calls_per_s": round(len(lat) / sum(lat), 1)}), flush=True)
        p.close()
    finally:
        stop.set()
        d.shutdown()
        w.shutdown()
        ctrl.stop()


def cmd_cache(args):
    from dlslime_b200 import PeerAgent
    from dlslime_b200.cache import CacheClient
    from dlslime_b200.cache.service import CacheServer
    from dlslime_b200.nanoctrl import start_local_nanoctrl

    ctrl = start_local_nanoctrl()
    srv = CacheServer(ctrl.url, slab_size=256 << 10, memory_size=max(64 << 20, 4 * args.length), alias="cache-agent:0")
    eng = PeerAgent(ctrl.url, alias="engine:0")
    try:
        buf = ctypes.create_string_buffer(args.length)
        eng.register_memory_region("kv", ctypes.addressof(buf), 0, args.length)
        cl = CacheClient(ctrl=ctrl.url, peer_agent=eng)
        cl.connect_to_server()
        put, get = [], []
        for _ in range(args.iters):
            t = time.perf_counter()
            m = cl.put("kv", [(0, args.length)])
            put.append(time.perf_counter() - t)
            t = time.perf_counter()
            cl.get("kv", eng.alias, m["version"])
            get.append(time.perf_counter() - t)
            cl.delete(eng.alias, m["version"])
        print(json.dumps({"bench": "cache_put_get", "bytes": args.length, "slabs": len(m["slab_ids"]),
                          "put_p50_ms": round(pct(put, 0.5) * 1e3, 3), "get_p50_ms": round(pct(get, 0.5) * 1e3, 3),
                          "put_mb_s": round(args.length / pct(put, 0.5) / 1e6, 1), "get_mb_s": round(args.length / pct(get, 0.5) / 1e6, 1)}), flush=True)
    finally:
        eng.shutdown()
        srv.stop()
        ctrl.stop()


def cmd_torch(args):
    import torch
    import torch.distributed as dist

    import dlslime_b200.torch_backend  # noqa: F401  (registers the backend)

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("dlslime")
    rank = dist.get_rank()
    for size in [int(s) for s in args.sizes.split(",")]:
        t = torch.zeros(size, dtype=torch.uint8)
        for _ in range(5):
            dist.send(t, 1) if rank == 0 else dist.recv(t, 0)
        t0 = time.perf_counter()
        for _ in range(args.iters):
            dist.send(t, 1) if rank == 0 else dist.recv(t, 0)
        dt = time.perf_counter() - t0
        if rank == 1:
            print(json.dumps({"bench": "torch_dist_sendrecv", "backend": "dlslime", "bytes": size, "us_per_msg": round(dt / args.iters * 1e6, 1),
                              "mb_s": round(size * args.iters / dt / 1e6, 1)}), flush=True)
    os._exit(0)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["io", "sendrecv", "rpc", "cache", "torch"])
    ap.add_argument("--transport", default="tcp", choices=["tcp", "rdma"])
    ap.add_argument("--sizes", default=None, help="default: 4096,65536,1048576,16777216 (rpc: 64,4096,65536,1048576, its slots hold 2 MiB)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--concurrency", type=int, default=1, help="io: operations kept in flight per iteration")
    ap.add_argument("--qp", type=int, default=2)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--length", type=int, default=16 << 20)
    a = ap.parse_args()
    if a.sizes is None:
        a.sizes = "64,4096,65536,1048576" if a.cmd == "rpc" else "4096,65536,1048576,16777216"
    {"io": cmd_io, "sendrecv": cmd_sendrecv, "rpc": cmd_rpc, "cache": cmd_cache, "torch": cmd_torch}[a.cmd](a)
