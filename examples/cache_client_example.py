#!/usr/bin/env python3
"""DLSlimeCache: store bytes of a local region in a cache service and read them back.

    python examples/cache_client_example.py          # control plane + cache service started in this process
    # or against running services:
    #   python -m dlslime_b200.nanoctrl start
    #   python -m dlslime_b200.cache start --ctrl http://127.0.0.1:3000 --memory-size 1G
    python examples/cache_client_example.py --ctrl http://127.0.0.1:3000

Same flow as the reference's examples/python/cache_client_example.py: ask the service for its PeerAgent, connect,
store a manifest (which allocates slabs), write the bytes into the cache region, query the manifest back, read.
"""
import argparse
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200 import PeerAgent  # noqa: E402
from dlslime_b200.cache import CacheClient  # noqa: E402
from dlslime_b200.cache.service import CacheServer  # noqa: E402
from dlslime_b200.nanoctrl import start_local_nanoctrl  # noqa: E402


def main(args):
    local = srv = None
    ctrl = args.ctrl
    if ctrl is None:
        local = start_local_nanoctrl()
        ctrl = local.url
        srv = CacheServer(ctrl, slab_size=256 << 10, memory_size=64 << 20, alias="cache-agent:0")
    engine = PeerAgent(ctrl, alias="engine:0")
    try:
        n = args.length
        payload = bytes(i % 251 for i in range(n))
        buf = ctypes.create_string_buffer(payload, n)
        engine.register_memory_region("kv", ctypes.addressof(buf), 0, n)
        client = CacheClient(ctrl=ctrl, peer_agent=engine)
        info = client.connect_to_server()
        print(f"connected: server_peer_agent_id={info['peer_agent_id']} cache_mr={info['cache_mr_name']} slab={info['slab_size']}")
        manifest = client.put("kv", [(0, n)])
        print(f"stored: version={manifest['version']} slabs={manifest['slab_ids']} bytes={manifest['total_bytes']}")
        ctypes.memset(ctypes.addressof(buf), 0, n)
        client.get("kv", engine.alias, manifest["version"])
        assert buf.raw == payload, "payload mismatch after reading back from the cache"
        assert client.delete(engine.alias, manifest["version"])
        print("read back and verified; entry deleted")
    finally:
        engine.shutdown()
        if srv is not None:
            srv.stop()
        if local is not None:
            local.stop()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctrl", default=None)
    ap.add_argument("--length", type=int, default=640 * 1024)
    main(ap.parse_args())
