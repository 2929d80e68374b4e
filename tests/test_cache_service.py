"""DLSlimeCache service + client over the control plane: HTTP contract, put/get of real bytes, discovery."""
import ctypes
import json
import urllib.error
import urllib.request

import pytest

from dlslime_b200._slime_c import Assignment
from dlslime_b200.cache import CacheClient, CacheHttpServer, CacheServer, CacheService, discover_cache_url, get_json, post_json
from dlslime_b200.nanoctrl import NanoCtrlClient, start_local_nanoctrl
from dlslime_b200.peer_agent import PeerAgent

K = 1024


def test_http_contract_without_a_peer_agent():
    http = CacheHttpServer(CacheService(slab_size=128 * K, memory_size=512 * K)).start()
    try:
        assert get_json(http.url, "/healthz") == {"ok": True}
        assert get_json(http.url, "/stats")["num_slabs"] == 4
        m = post_json(http.url, "/store", {"peer_agent_id": "e", "assignments": [{"mr_key": 1, "remote_mr_key": 2, "target_offset": 10, "source_offset": 0, "length": 200 * K}]})
        assert m["version"] == 1 and m["slab_ids"] == [0, 1] and m["total_bytes"] == 200 * K
        assert [(a["target_offset"], a["source_offset"], a["length"]) for a in m["assignments"]] == [(10, 0, 128 * K), (10 + 128 * K, 128 * K, 72 * K)]
        assert post_json(http.url, "/query", {"peer_agent_id": "e", "version": 1}) == m
        with pytest.raises(RuntimeError, match="HTTP 404"):
            post_json(http.url, "/query", {"peer_agent_id": "e", "version": 9})
        with pytest.raises(RuntimeError, match="HTTP 400"):
            post_json(http.url, "/store", {"peer_agent_id": "", "assignments": []})
        with pytest.raises(RuntimeError, match="HTTP 503"):
            get_json(http.url, "/peer-agent")
        assert post_json(http.url, "/delete", {"peer_agent_id": "e", "version": 1}) == {"deleted": True}
        assert post_json(http.url, "/delete", {"peer_agent_id": "e", "version": 1}) == {"deleted": False}
        req = urllib.request.Request(http.url + "/store", data=b"not json", method="POST")
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.build_opener(urllib.request.ProxyHandler({})).open(req)
        assert e.value.code == 400 and "error" in json.loads(e.value.read())
    finally:
        http.stop()


def test_put_get_roundtrip_through_the_control_plane():
    ctrl = start_local_nanoctrl()
    srv = CacheServer(ctrl.url, slab_size=128 * K, memory_size=8 * 128 * K, alias="cache-agent:0", scope="c")
    eng = PeerAgent(ctrl.url, alias="engine-a", scope="c")
    try:
        assert discover_cache_url(ctrl.url, scope="c") == srv.url
        ent = NanoCtrlClient(ctrl.url, scope="c").get_entity_info("cache:0")
        assert ent["kind"] == "cache" and ent["endpoint"]["protocol"] == "http" and ent["endpoint"]["port"] == srv.http.port
        buf = ctypes.create_string_buffer(1 << 20)
        buf.raw = bytes(i % 253 for i in range(1 << 20))
        eng.register_memory_region("kv", ctypes.addressof(buf), 0, 1 << 20)
        cl = CacheClient(ctrl=ctrl.url, scope="c", peer_agent=eng)
        info = cl.connect_to_server()
        assert info["peer_agent_id"] == "cache-agent:0" and info["cache_mr_name"] == "cache" and info["memory_size"] == 8 * 128 * K
        m = cl.put("kv", [(4096, 300 * K), (800000, 1000)])
        assert m["slab_ids"] == [0, 1, 2, 3] and cl.stats()["used_slabs"] == 4
        # the manifest's source_offset is the offset inside the cache region: the bytes really are there
        first = m["assignments"][0]
        assert bytes(srv.service.cache_storage)[first["source_offset"]:first["source_offset"] + 16] == buf.raw[4096:4112]
        orig = buf.raw
        ctypes.memset(ctypes.addressof(buf), 0, 1 << 20)
        cl.get("kv", "engine-a", m["version"])
        assert buf.raw[4096:4096 + 300 * K] == orig[4096:4096 + 300 * K] and buf.raw[800000:801000] == orig[800000:801000]
        assert buf.raw[:4096] == bytes(4096)
        assert cl.delete("engine-a", m["version"]) and cl.stats()["used_slabs"] == 0
        assert cl.store([Assignment(0, 0, 0, 0, 64)], peer_agent_id="other")["peer_agent_id"] == "other"
    finally:
        eng.shutdown()
        srv.stop()
        ctrl.stop()


def test_http_service_survives_malformed_requests():
    """Seeded junk on every route (wrong types, huge and negative numbers, raw bytes, wrong methods): always a JSON answer
    with a sensible status, no slab leaks, and the service still works afterwards."""
    import random

    http = CacheHttpServer(CacheService(slab_size=128 * K, memory_size=1024 * K)).start()
    try:
        rnd = random.Random(9)
        keys = ["peer_agent_id", "assignments", "version", "mr_key", "remote_mr_key", "target_offset", "source_offset", "length", "x"]
        def junk(d=0):
            k = rnd.randint(0, 7 if d < 3 else 4)
            if k == 0: return None
            if k == 1: return rnd.choice([True, False])
            if k == 2: return rnd.choice([-1, 0, 1, 2**31, 2**63, 2**64, -2**63, 300 * K])
            if k == 3: return rnd.random() * 1e6
            if k == 4: return rnd.choice(["", "e", "peer\n", "é"])
            if k == 5: return [junk(d + 1) for _ in range(rnd.randint(0, 3))]
            return {rnd.choice(keys): junk(d + 1) for _ in range(rnd.randint(0, 6))}
        codes = {}
        opener = urllib.request.build_opener(urllib.request.ProxyHandler({}))
        for i in range(300):
            route = rnd.choice(["/store", "/query", "/delete", "/stats", "/healthz", "/peer-agent", "/zzz"])
            kind = rnd.random()
            body = json.dumps(junk()).encode() if kind < 0.8 else bytes(rnd.randrange(256) for _ in range(rnd.randint(0, 30)))
            req = urllib.request.Request(http.url + route, data=body, method=rnd.choice(["POST", "POST", "GET"]))
            try:
                with opener.open(req, timeout=5) as r:
                    code, text = r.status, r.read()
            except urllib.error.HTTPError as e:
                code, text = e.code, e.read()
            codes[code] = codes.get(code, 0) + 1
            assert code in (200, 400, 404, 405, 501, 503), (route, body, code, text[:200])
            json.loads(text)
        st = get_json(http.url, "/stats")
        assert st["num_slabs"] == 8 and st["used_slabs"] + st["free_slabs"] == 8
        m = post_json(http.url, "/store", {"peer_agent_id": "after", "assignments": [{"mr_key": 1, "remote_mr_key": 2, "target_offset": 0, "source_offset": 0, "length": 10}]})
        assert post_json(http.url, "/query", {"peer_agent_id": "after", "version": m["version"]}) == m
    finally:
        http.stop()


def test_concurrent_engines_put_get_delete_and_no_slab_leaks():
    """Four engines, each with its own PeerAgent, put / get / delete random extents at the same time: every read-back is
    byte exact and the directory ends with every slab free."""
    import random
    import threading

    from dlslime_b200.peer_agent import PeerAgent

    ctrl = start_local_nanoctrl()
    srv = CacheServer(ctrl.url, slab_size=128 * K, memory_size=16 << 20, alias="cache-agent:0")
    errs = []

    def engine(k):
        ag = None
        try:
            ag = PeerAgent(ctrl.url, alias=f"engine:{k}")
            rnd = random.Random(k)
            n = 1 << 20
            buf = ctypes.create_string_buffer(rnd.randbytes(n), n)
            orig = buf.raw
            ag.register_memory_region("kv", ctypes.addressof(buf), 0, n)
            cl = CacheClient(ctrl=ctrl.url, peer_agent=ag)
            cl.connect_to_server()
            live = []

            def read_back(v, o, ln):
                ctypes.memset(ctypes.addressof(buf) + o, 0, ln)
                cl.get("kv", ag.alias, v)
                assert buf.raw[o:o + ln] == orig[o:o + ln], (k, v)
                assert cl.delete(ag.alias, v)

            for _ in range(10):
                off, ln = rnd.randrange(0, n - 300_000), rnd.choice([1, 4096, 128 * K, 200_000, 300_000])
                live.append((cl.put("kv", [(off, ln)])["version"], off, ln))
                if len(live) > 2 and rnd.random() < 0.5:
                    read_back(*live.pop(rnd.randrange(len(live))))
            for item in live:
                read_back(*item)
        except Exception as e:  # noqa: BLE001
            errs.append((k, repr(e)))
        finally:
            if ag is not None:
                ag.shutdown()

    try:
        ths = [threading.Thread(target=engine, args=(k,)) for k in range(4)]
        [t.start() for t in ths]
        [t.join(120) for t in ths]
        assert not errs and not any(t.is_alive() for t in ths), errs
        st = srv.service.stats()
        assert st.used_slabs == 0 and st.free_slabs == st.num_slabs and st.num_assignment_entries == 0
    finally:
        srv.stop()
        ctrl.stop()
