"""Embedded key-value store (Redis semantics, fake clock) and the NanoCtrl HTTP contract."""
import json
import threading
import time

import pytest

from dlslime_b200 import _slime_c as c
from dlslime_b200.nanoctrl import NanoCtrlClient, NanoCtrlError, RespClient, RespError, start_local_nanoctrl

KvStore = c.ctrl.KvStore


def test_ttl_expiry_with_injected_clock():
    kv = KvStore()
    now = [1_000_000]
    kv.set_clock(lambda: now[0])
    kv.set("k", "v", px=5000)
    assert kv.get("k") == "v" and 0 < kv.pttl("k") <= 5000
    now[0] += 4999
    assert kv.exists("k")
    now[0] += 2
    assert kv.get("k") is None and kv.pttl("k") == -2
    kv.hset("h", {"a": "1"})
    kv.expire("h", 60)
    now[0] += 59_000
    assert kv.pexpire("h", 60_000)  # heartbeat renews
    now[0] += 59_000
    assert kv.hgetall("h") == {"a": "1"}
    now[0] += 2_000
    assert kv.hgetall("h") == {} and not kv.pexpire("h", 1000)


def test_set_nx_incr_types_and_scan():
    kv = KvStore()
    assert kv.set("a", "1", nx=True) and not kv.set("a", "2", nx=True)
    assert kv.incr("a") == 2 and kv.incr("ctr", 5) == 5
    kv.lpush("l", "x")
    with pytest.raises(RuntimeError, match="WRONGTYPE"):
        kv.incr("l")
    for i in range(25):
        kv.set(f"mr:A:{i}", "x")
    assert len(kv.keys("mr:A:*")) == 25 and kv.keys("mr:A:1?") == [f"mr:A:1{i}" for i in range(10)]
    seen, cursor = [], 0
    while True:
        cursor, ks = kv.scan(cursor, "mr:*", 7)
        seen += ks
        if cursor == 0:
            break
    assert sorted(seen) == sorted(kv.keys("mr:*"))
    assert KvStore.glob_match("exchange:*:B", "exchange:A:B") and not KvStore.glob_match("a[0-9]c", "abc") and KvStore.glob_match("a[0-9]c", "a7c")


def test_lists_and_blocking_pop_wakeup():
    kv = KvStore()
    assert kv.blpop(["inbox"], 0.05) is None
    got = []
    t = threading.Thread(target=lambda: got.append(kv.blpop(["inbox"], 2.0)))
    t.start()
    time.sleep(0.05)
    kv.lpush("inbox", "a", "b")  # LPUSH a b -> list is [b, a]
    t.join(2)
    assert got == [("inbox", "b")] and kv.lrange("inbox", 0, -1) == ["a"] and kv.llen("inbox") == 1


def test_streams_ids_maxlen_and_blocking_read():
    kv = KvStore()
    i1 = kv.xadd("s", {"type": "connect_peer", "peer": "B"})
    i2 = kv.xadd("s", {"type": "qp_ready"})
    assert i1 < i2 or tuple(map(int, i1.split("-"))) < tuple(map(int, i2.split("-")))
    res = kv.xread({"s": "0-0"})
    assert [e[1]["type"] for e in res[0][1]] == ["connect_peer", "qp_ready"]
    assert kv.xread({"s": i2}) == [] and kv.xread({"s": "$"}, block=20) == []
    with pytest.raises(RuntimeError):
        kv.xadd("s", {"a": "b"}, id="0-1")  # ids must increase
    for n in range(20):
        kv.xadd("s", {"n": str(n)}, maxlen=5)
    assert kv.xlen("s") == 5
    out = []
    t = threading.Thread(target=lambda: out.append(kv.xread({"late": "0-0"}, block=2000)))
    t.start()
    time.sleep(0.05)
    kv.xadd("late", {"x": "1"})
    t.join(2)
    assert out[0][0][1][0][1] == {"x": "1"}


def test_publish_subscribe():
    kv = KvStore()
    got = []
    tok = kv.subscribe("nano_events:*", lambda ch, msg: got.append((ch, msg)))
    assert kv.publish("nano_events:service_update", "hello") == 1
    kv.unsubscribe(tok)
    assert kv.publish("nano_events:service_update", "again") == 0 and got == [("nano_events:service_update", "hello")]


@pytest.fixture()
def ctrl():
    n = start_local_nanoctrl()
    yield n
    n.stop()


def test_resp_front_end_speaks_redis(ctrl):
    r = RespClient("127.0.0.1", ctrl.resp_port)
    assert r.ping() and r.set("k", "v", ex=10) and r.get("k") == "v" and 0 < r.ttl("k") <= 10
    assert r.hset("h", mapping={"a": 1, "b": 2}) == 2 and r.hgetall("h") == {"a": "1", "b": "2"}
    assert r.lpush("l", "x") == 1 and r.blpop("l", 1) == ("l", "x") and r.blpop("l", 0.05) is None
    r.xadd("s", {"f": "v"}, maxlen=10)
    assert r.xread({"s": "0-0"}, block=10)[0][1][0][1] == {"f": "v"}
    assert r.mget(["k", "missing"]) == ["v", None] and r.delete("k", "h") == 2
    with pytest.raises(RespError):
        r.execute("NOSUCHCOMMAND")
    with pytest.raises(RespError, match="WRONGTYPE"):
        r.execute("INCR", "s")
    # the in-process handle and the socket see the same data
    assert ctrl.store.xlen("s") == 1


def test_http_routes_and_error_codes(ctrl):
    cl = NanoCtrlClient(ctrl.url, scope="t")
    assert cl.check_connection()
    rsp = cl.register_peer("10.0.0.1", alias="A", device="tcp0", ib_port=1, link_type="TCP", resource={"nics": []})
    assert rsp["status"] == "ok" and rsp["name"] == "A" and rsp["redis_address"].endswith(f":{ctrl.resp_port}")
    with pytest.raises(NanoCtrlError) as e:
        cl.register_peer("10.0.0.1", alias="A")
    assert e.value.status == 409
    auto = [cl.register_peer("10.0.0.2")["name"] for _ in range(2)]
    assert auto == ["agent-1", "agent-2"]
    agents = {a["name"]: a for a in cl.query_peers()}
    assert set(agents) == {"A", "agent-1", "agent-2"} and agents["A"]["link_type"] == "TCP" and agents["A"]["resource"] == {"nics": []}
    assert ctrl.store.pttl("t:agent:A") > 0  # 60 s lease
    assert cl.heartbeat_peer("A") == "ok" and cl.heartbeat_peer("ghost") == "not_found"
    # scope isolation
    assert NanoCtrlClient(ctrl.url, scope="other").query_peers() == []
    # memory regions
    cl.register_mr("A", "kv", 0x7F00, 4096, 77)
    assert cl.get_mr_info("B", "A", "kv") == {"addr": 0x7F00, "length": 4096, "rkey": 77, "lkey": 0}
    assert cl.get_mr_info("B", "A", "nope") is None
    assert cl.get_redis_url() == f"redis://127.0.0.1:{ctrl.resp_port}"
    status, body = ctrl._srv.handle("POST", "/nope", "{}")
    assert status == 404 and json.loads(body)["status"] == "error"
    status, body = ctrl._srv.handle("POST", "/heartbeat", "not json")
    assert status == 400


def test_desired_topology_streams_and_cleanup_notifications(ctrl):
    cl = NanoCtrlClient(ctrl.url)
    for name in ("A", "B", "C"):
        cl.register_peer("10.0.0.1", alias=name)
    cl.set_desired_topology("A", ["B"], symmetric=True)
    cl.set_desired_topology("C", ["A"])
    kv = ctrl.store
    assert json.loads(kv.get("spec:topology:A"))["target_peers"] == ["B"]
    assert json.loads(kv.get("spec:topology:B"))["target_peers"] == ["A"]  # symmetric back-edge
    a_msgs = kv.xrange("stream:A")
    assert [m[1]["peer"] for m in a_msgs] == ["B"] and a_msgs[0][1]["type"] == "connect_peer"
    assert [m[1]["peer"] for m in kv.xrange("stream:B")] == ["A"]
    kv.set("exchange:A:B", "x")
    kv.set("mr:A:kv", "{}")
    cl.cleanup_peer("A")
    assert not kv.exists("agent:A") and kv.keys("exchange:*") == [] and kv.keys("mr:A:*") == []
    # B (targeted by A, and targeting A) and C (targeting A) are told; A itself is not
    for peer in ("B", "C"):
        assert json.loads(kv.lpop(f"inbox:{peer}")) == {"type": "cleanup", "peer": "A"}
    assert kv.llen("inbox:A") == 0


def test_entities_events_and_lease(ctrl):
    cl = NanoCtrlClient(ctrl.url)
    events = []
    ctrl.store.subscribe("nano_events:service_update", lambda ch, m: events.append(json.loads(m)))
    cl.register("cache:0", "cache", endpoint={"host": "h", "port": 1, "protocol": "http"}, metadata={"p2p_host": "h"})
    info = cl.get_entity_info("cache:0")
    assert info["kind"] == "cache" and info["id"] == "cache:0" and info["endpoint"]["port"] == 1
    assert [e["entity_id"] for e in cl.list_entities(kind="cache")] == ["cache:0"] and cl.list_entities(kind="router") == []
    assert cl.heartbeat("cache:0") == "ok"
    cl.unregister("cache:0")
    assert cl.unregister("cache:0")["status"] == "ok"  # absent is still ok
    assert cl.get_entity_info("cache:0") is None
    assert [(e["event_type"], e["revision"]) for e in events] == [("ADD", 1), ("REMOVE", 2)]


def test_http_routes_survive_malformed_requests():
    """Seeded junk on every route (wrong types, truncated JSON, raw bytes, wrong methods): the server always answers with
    JSON and a sensible status, never hangs up, and still serves afterwards."""
    import random
    import urllib.error
    import urllib.request

    ctrl = start_local_nanoctrl()
    routes = ["/heartbeat", "/start_peer_agent", "/query", "/cleanup", "/v1/desired_topology/x", "/register_mr", "/get_mr_info",
              "/register", "/unregister", "/get_entity_info", "/list_entities", "/get_redis_address", "/nope"]
    keys = ["entity_type", "entity_id", "kind", "endpoint", "metadata", "agent_name", "alias", "address", "target_peers", "mr_name",
            "addr", "length", "rkey", "src", "dst", "scope", "symmetric", "resource", "name_prefix", "x"]
    rnd = random.Random(5)

    def junk(depth=0):
        k = rnd.randint(0, 7 if depth < 3 else 4)
        if k == 0:
            return None
        if k == 1:
            return rnd.choice([True, False])
        if k == 2:
            return rnd.randint(-2 ** 40, 2 ** 40)
        if k == 3:
            return rnd.random() * 1e6
        if k == 4:
            return "".join(chr(rnd.choice([34, 92, 10, 0x1F600, 65, 0xE9, 0])) for _ in range(rnd.randint(0, 6)))
        if k == 5:
            return [junk(depth + 1) for _ in range(rnd.randint(0, 3))]
        return {rnd.choice(keys): junk(depth + 1) for _ in range(rnd.randint(0, 5))}

    try:
        for _ in range(500):
            route, kind = rnd.choice(routes), rnd.random()
            if kind < 0.7:
                body = json.dumps(junk()).encode()
            elif kind < 0.85:
                body = bytes(rnd.randrange(256) for _ in range(rnd.randint(0, 40)))
            else:
                body = json.dumps(junk()).encode()[: rnd.randint(0, 10)]
            req = urllib.request.Request(ctrl.url + route, data=body, headers={"Content-Type": "application/json"},
                                         method=rnd.choice(["POST", "POST", "GET", "PUT"]))
            try:
                with urllib.request.urlopen(req, timeout=5) as r:
                    code, text = r.status, r.read()
            except urllib.error.HTTPError as e:
                code, text = e.code, e.read()
            assert code in (200, 400, 404, 405, 409, 500), (route, body, code)
            json.loads(text)
        client = NanoCtrlClient(ctrl.url)
        assert client.check_connection()
        assert client.register("after:1", "probe")["status"] == "ok" and client.get_entity_info("after:1")["kind"] == "probe"
    finally:
        ctrl.stop()


def test_entities_expire_without_heartbeat_on_an_injected_clock():
    """Through the HTTP routes: an entity lives ENTITY_TTL_SECS after its last heartbeat, a heartbeat for one that is gone
    says not_found (the caller re-registers), and listings show only what is alive."""
    ctrl = start_local_nanoctrl()
    try:
        now = [ctrl.store.now_ms()]
        ctrl.store.set_clock(lambda: now[0])
        cl = NanoCtrlClient(ctrl.url, scope="ttl")
        for i in range(3):
            assert cl.register(f"svc:{i}", "worker")["status"] == "ok"
        assert sorted(e["entity_id"] for e in cl.list_entities(kind="worker")) == ["svc:0", "svc:1", "svc:2"]
        now[0] += (c.ctrl.ENTITY_TTL_SECS - 1) * 1000
        assert cl.heartbeat("svc:0") == "ok"
        now[0] += 2_000
        assert sorted(e["entity_id"] for e in cl.list_entities(kind="worker")) == ["svc:0"]
        assert cl.heartbeat("svc:1") == "not_found" and cl.get_entity_info("svc:2") is None
        assert cl.register("svc:1", "worker")["status"] == "ok" and cl.heartbeat("svc:1") == "ok"
    finally:
        ctrl.stop()
