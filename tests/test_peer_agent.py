"""PeerAgent over the in-process control plane and TCP endpoints: handshake, named I/O translation,
region lifecycle, scope isolation, peer exit, dropped handshake messages, lease expiry."""
import ctypes
import json
import time

import pytest

from dlslime_b200.nanoctrl import start_local_nanoctrl
from dlslime_b200.peer_agent import PeerAgent


@pytest.fixture()
def ctrl():
    n = start_local_nanoctrl()
    yield n
    n.stop()


def _region(agent, name, size=1 << 16, fill=None):
    b = ctypes.create_string_buffer(size)
    if fill is not None:
        b.raw = bytes((fill + i) % 251 for i in range(size))
    agent.register_memory_region(name, ctypes.addressof(b), 0, size)
    return b


def test_handshake_named_io_and_mirror_connection(ctrl):
    a, b = PeerAgent(ctrl.url, alias="A", scope="s"), PeerAgent(ctrl.url, alias="B", scope="s")
    try:
        ba, bb = _region(a, "kv", fill=1), _region(b, "kv", fill=9)
        conn = a.connect_to("B").wait(10)
        assert conn.is_connected() and conn.conn_id == "A:tcp0:port1->B:tcp0:port1#qp1" and (conn.local_nic, conn.remote_nic) == ("tcp0", "tcp0")
        assert a.list_agents() == ["A", "B"] and a.list_mem_keys("B") == ["kv"]
        # (region, local_off, remote_off, len): local bytes [0,5000) land at remote offset 100
        assert a.write("B", [("kv", 0, 100, 5000)]).wait(10) == 0 and bb.raw[100:5100] == ba.raw[:5000]
        # 5-tuple names both regions; the peer answers on its mirrored connection
        mirror = b.query_connection("A")
        assert mirror is not None and mirror.wait(5).is_connected()
        assert b.read("A", ("kv", "kv", 30000, 7, 1000)).wait(10) == 0 and bb.raw[30000:31000] == ba.raw[7:1007]
        assert a.write_with_imm("B", [("kv", 0, 0, 16)], imm_data=42).wait(10) == 0
        f = b.imm_recv("A")
        assert f.wait(10) == 0 and f.imm_data() == 42
        with pytest.raises(ValueError):
            a.connect_to("A")
        with pytest.raises(KeyError):
            a.write("B", [("nope", 0, 0, 1)])
    finally:
        a.shutdown()
        b.shutdown()


def test_named_tuple_translation_is_pinned(ctrl):
    """(local_region, remote_region, local_off, remote_off, len) -> (lh, rh, remote_off, local_off, len)."""
    a, b = PeerAgent(ctrl.url, alias="A"), PeerAgent(ctrl.url, alias="B")
    try:
        keep = [_region(a, "x"), _region(a, "y"), _region(b, "x"), _region(b, "y")]  # registered memory must stay alive
        a.connect_to("B").wait(10)
        conn = a._get_connection("B")
        lh, rh = a.get_handle(conn, "y"), a.get_handle(conn, "x", remote=True)
        assert a._endpoint_assign(conn, ("y", "x", 16, 8, 32)) == (lh, rh, 8, 16, 32)
        assert a._endpoint_assign(conn, ("x", 16, 8, 32))[2:] == (8, 16, 32)
        assert a._maybe_endpoint_assign(conn, [(1, 2, 3, 4, 5)]) == [(1, 2, 3, 4, 5)]  # handle tuples pass through
    finally:
        a.shutdown()
        b.shutdown()


def test_region_publication_unregister_and_cache_validation(ctrl):
    a, b = PeerAgent(ctrl.url, alias="A"), PeerAgent(ctrl.url, alias="B")
    try:
        ba = _region(a, "kv", fill=3)
        bb = _region(b, "kv")
        kv = ctrl.store
        rec = json.loads(kv.get("mr:B:kv"))
        assert rec == json.loads(kv.get("mr:B:kv:tcp0:1:TCP")) and rec["agent_name"] == "B" and rec["length"] == 1 << 16 and rec["lkey"] == 0
        a.connect_to("B").wait(10)
        assert a.write("B", [("kv", 0, 0, 64)]).wait(10) == 0
        # B replaces the region by a bigger one at a new address: A notices through cache validation
        big = ctypes.create_string_buffer(1 << 17)
        assert b.unregister_memory_region("kv") and not b.unregister_memory_region("kv")
        assert kv.get("mr:B:kv") is None and b.list_mem_keys() == []
        b.register_memory_region("kv", ctypes.addressof(big), 0, 1 << 17)
        assert a.write("B", [("kv", 0, 100000, 64)]).wait(10) == 0 and big.raw[100000:100064] == ba.raw[:64]
        del bb
    finally:
        a.shutdown()
        b.shutdown()


def test_scopes_are_isolated_and_alias_conflict_is_fatal(ctrl):
    a = PeerAgent(ctrl.url, alias="A", scope="one")
    b = PeerAgent(ctrl.url, alias="A", scope="two")  # same alias, other scope: fine
    try:
        assert a.list_agents() == ["A"] and b.list_agents() == ["A"]
        with pytest.raises(RuntimeError, match="already registered"):
            PeerAgent(ctrl.url, alias="A", scope="one")
        with pytest.raises(KeyError):
            a.connect_to("B")
        auto = PeerAgent(ctrl.url, scope="one")
        assert auto.alias.startswith("agent-")
        auto.shutdown()
    finally:
        a.shutdown()
        b.shutdown()


def test_peer_shutdown_drops_the_connection_and_fails_waiters(ctrl):
    a, b = PeerAgent(ctrl.url, alias="A"), PeerAgent(ctrl.url, alias="B")
    try:
        keep = [_region(a, "kv"), _region(b, "kv")]  # registered memory must stay alive
        a.connect_to("B").wait(10)
        b.query_connection("A").wait(5)
        waiter = b.imm_recv("A")
        a.shutdown()
        assert waiter.wait(5) == 403  # the cleanup notice shut B's endpoint down; nobody hangs
        deadline = time.monotonic() + 5
        while b.get_connections() and time.monotonic() < deadline:
            time.sleep(0.02)
        assert b.get_connections() == {}
        assert not ctrl.store.exists("agent:A") and ctrl.store.keys("mr:A:*") == []
        # and A can come back under the same alias and reconnect
        a2 = PeerAgent(ctrl.url, alias="A")
        keep.append(_region(a2, "kv"))
        a2.connect_to("B").wait(10)
        assert a2.write("B", [("kv", 0, 0, 8)]).wait(10) == 0
        a2.shutdown()
    finally:
        a.shutdown()
        b.shutdown()


def test_dropped_handshake_message_times_out_cleanly(ctrl):
    a, b = PeerAgent(ctrl.url, alias="A"), PeerAgent(ctrl.url, alias="B")
    try:
        b._mailbox.message_filter = lambda msg: msg.get("type") != "qp_ready"  # B never sees A's announcement
        conn = a.connect_to("B")
        with pytest.raises(TimeoutError):
            conn.wait(0.5)
        assert conn.state in ("pending", "connecting")
    finally:
        a.shutdown()
        b.shutdown()


def test_expired_lease_is_renewed_by_re_registration(ctrl):
    a = PeerAgent(ctrl.url, alias="A")
    try:
        keep = _region(a, "kv")
        ctrl.store.delete("agent:A")  # what a missed lease looks like to the control plane
        a._heartbeat_once()
        assert ctrl.store.exists("agent:A") and json.loads(ctrl.store.hget("agent:A", "memory_keys")) == ["kv"]
    finally:
        a.shutdown()


def test_obs_reporter_snapshot_and_stopped_marker(ctrl):
    from dlslime_b200 import _slime_c as c

    c.obs_set_enabled_for_test(True)
    c.obs_reset_for_test()
    a, b = PeerAgent(ctrl.url, alias="A", enable_obs=True), PeerAgent(ctrl.url, alias="B")
    try:
        keep = [_region(a, "kv"), _region(b, "kv")]  # registered memory must stay alive
        a.connect_to("B").wait(10)
        assert a.write("B", [("kv", 0, 0, 4096)]).wait(10) == 0
        snap = a._obs.report_once()
        assert snap["schema_version"] == 1 and snap["peer_id"] == "A" and snap["summary"]["completed_bytes_total"] >= 4096
        assert snap["connections"][0]["peer"] == "B" and snap["connections"][0]["connected"]
        assert any(n["kind"] == "tcp" for n in snap["nics"])
        stored = json.loads(ctrl.store.get("obs:peer:A"))
        assert stored["session_id"] == snap["session_id"] and 0 < ctrl.store.pttl("obs:peer:A") <= 180_000
    finally:
        a.shutdown()
        b.shutdown()
        c.obs_reset_for_test()
        c.obs_set_enabled_for_test(False)
    stopped = json.loads(ctrl.store.get("obs:peer:A"))
    assert stopped["status"] == "stopped" and ctrl.store.pttl("obs:peer:A") <= 15_000


def test_concurrent_full_mesh_then_rejoin_after_exit_and_after_crash(ctrl):
    """Five agents connect to each other at the same time from five threads; every ordered pair writes. Then one agent
    leaves cleanly and comes back under its alias, and later dies without any cleanup and comes back again: both times the
    others shake hands anew (a peer that announces other endpoints than the ones a link is connected to has restarted)."""
    import threading

    n = 5
    agents, bufs = [], []
    for i in range(n):
        a = PeerAgent(ctrl.url, alias=f"n{i}", scope="mesh")
        b = ctypes.create_string_buffer(bytes([i + 1]) * 4096, 4096)
        a.register_memory_region("m", ctypes.addressof(b), 0, 4096)
        agents.append(a), bufs.append(b)
    try:
        errs = []

        def connect_all(i):
            try:
                for c in [agents[i].connect_to(f"n{j}") for j in range(n) if j != i]:
                    c.wait(20)
            except Exception as e:  # noqa: BLE001
                errs.append((i, repr(e)))

        ths = [threading.Thread(target=connect_all, args=(i,)) for i in range(n)]
        [t.start() for t in ths]
        [t.join(60) for t in ths]
        assert not errs and not any(t.is_alive() for t in ths)
        futs = [(i, j, agents[i].write(f"n{j}", [("m", 2048, 16 * i, 16)])) for i in range(n) for j in range(n) if i != j]
        assert all(f.wait(20) == 0 for _, _, f in futs)
        assert all(bufs[j].raw[16 * i:16 * i + 16] == bytes([i + 1]) * 16 for i in range(n) for j in range(n) if i != j)
        # the posted topology is cumulative, so everyone this agent connected to is told when it leaves
        spec = json.loads(ctrl.store.get("mesh:spec:topology:n2"))
        assert sorted(spec["target_peers"]) == ["n0", "n1", "n3", "n4"]

        def rejoin(fill):
            b = ctypes.create_string_buffer(bytes([fill]) * 4096, 4096)
            agents[2] = PeerAgent(ctrl.url, alias="n2", scope="mesh")
            bufs[2] = b
            agents[2].register_memory_region("m", ctypes.addressof(b), 0, 4096)
            for i in (0, 1, 3):
                c1, c2 = agents[i].connect_to("n2"), agents[2].connect_to(f"n{i}")
                # the newcomer's side first: once it is up, the old agent has at least begun to replace a link that it
                # still believed connected (after a crash nothing told it otherwise), and its handle waits for the new one
                c2.wait(20)
                c1.wait(20)
                assert agents[i].write("n2", [("m", 2048, 16 * i, 16)]).wait(20) == 0
                assert b.raw[16 * i:16 * i + 16] == bytes([i + 1]) * 16
                assert agents[2].write(f"n{i}", [("m", 2048, 16 * 2, 16)]).wait(20) == 0
                assert bufs[i].raw[32:48] == bytes([fill]) * 16

        agents[2].shutdown()  # clean exit: the others get a cleanup notice
        time.sleep(0.5)
        rejoin(77)
        # a crash: no cleanup call, no key removed by the agent itself; its lease just runs out
        dead = agents[2]
        dead._client.cleanup_peer = lambda *a, **k: None
        dead._store_delete_disabled = True
        dead._stop.set()
        dead._mailbox.stop()
        for c in list(dead._connections.values()):
            if c.endpoint is not None:
                c.endpoint.shutdown()
        ctrl.store.delete("mesh:agent:n2")
        time.sleep(0.3)
        rejoin(88)
    finally:
        for a in agents:
            try:
                a.shutdown()
            except Exception:
                pass


def test_names_that_share_memory_are_independent(ctrl):
    """Two logical regions on the same pointer and a window into it: all three are reachable by name from a peer, and
    unregistering one of the two full-size names leaves the other one working."""
    a, b = PeerAgent(ctrl.url, alias="A"), PeerAgent(ctrl.url, alias="B")
    try:
        src = _region(a, "src", 4096, fill=7)
        dst = ctypes.create_string_buffer(4096)
        b.register_memory_region("kv", ctypes.addressof(dst), 0, 4096)
        b.register_memory_region("kv_alias", ctypes.addressof(dst), 0, 4096)
        b.register_memory_region("kv_tail", ctypes.addressof(dst), 2048, 2048)
        a.connect_to("B").wait(10)
        b.connect_to("A").wait(10)
        assert a.write("B", [("src", "kv_alias", 0, 0, 100)]).wait(10) == 0 and dst.raw[:100] == src.raw[:100]
        assert a.write("B", [("src", "kv_tail", 100, 0, 50)]).wait(10) == 0 and dst.raw[2048:2098] == src.raw[100:150]
        assert b.unregister_memory_region("kv_alias") and sorted(b.list_mem_keys()) == ["kv", "kv_tail"]
        assert a.write("B", [("src", "kv", 200, 300, 10)]).wait(10) == 0 and dst.raw[300:310] == src.raw[200:210]
    finally:
        a.shutdown()
        b.shutdown()


def test_peer_that_only_speaks_exchange_keys_connects(ctrl):
    """Interop with the older handshake: the peer never sends ``qp_ready``; it publishes its endpoint description under
    ``exchange:{peer}:{me}`` and reads ours from ``exchange:{me}:{peer}:{conn_id}``."""
    import threading

    from dlslime_b200 import _slime_c
    from dlslime_b200.nanoctrl.client import NanoCtrlClient

    a = PeerAgent(ctrl.url, alias="A", scope="s")
    legacy = PeerAgent(ctrl.url, alias="OLD", scope="s")  # used for registration and its resource record only ...
    legacy._mailbox.message_filter = lambda msg: False      # ... it ignores every stream message, as an old peer would
    legacy._poll_exchange_keys = lambda store=None: 0       # and does not run the new fallback itself
    ep = _slime_c.TcpEndpoint()
    n = 1 << 16
    theirs = ctypes.create_string_buffer(n)
    ep.register_memory_region("kv", ctypes.addressof(theirs), 0, n)
    kv = ctrl.store
    try:
        ba = _region(a, "kv", fill=5)
        pending = a.connect_to("OLD")
        # the old peer: publish, then wait for A's key and connect
        kv.set("s:exchange:OLD:A", json.dumps(ep.endpoint_info()))
        deadline = time.time() + 10
        mine = None
        while time.time() < deadline and mine is None:
            keys = [k for k in kv.keys("s:exchange:A:OLD:*")]
            if keys:
                mine = json.loads(kv.get(keys[0]))
            time.sleep(0.02)
        assert mine is not None, "A never wrote its exchange key"
        assert json.loads(kv.get("s:exchange:A:OLD")) == mine
        assert ep.connect(mine) == 0
        conn = pending.wait(10)
        assert conn.is_connected()
        # data flows over the link that was completed from the exchange key (handles straight on the endpoint:
        # an old peer publishes no named memory keys either)
        link = a._get_connection("OLD")
        rh = link.endpoint.register_remote_memory_region("kv", ep.endpoint_info()["mr_info"]["kv"])
        lh = link.endpoint.get_mr_handle("kv")
        assert link.endpoint.write([(lh, rh, 128, 0, 4096)]).wait(10) == 0
        assert theirs.raw[128:128 + 4096] == ba.raw[:4096]
    finally:
        ep.shutdown()
        a.shutdown()
        legacy.shutdown()
