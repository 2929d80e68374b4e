"""SlimeRPC over PeerAgents on TCP endpoints: typed / raw / None results, remote exceptions, timeouts with
slot reclamation, back-pressure with more calls than slots, wire constants."""
import threading
import time

import pytest

from dlslime_b200 import _slime_c as c
from dlslime_b200.nanoctrl import start_local_nanoctrl
from dlslime_b200.peer_agent import PeerAgent
from dlslime_b200.rpc import MethodRegistry, RemoteRpcError, RpcError, RpcTimeoutError, method, proxy, serve, wait_all


class Calc:
    def __init__(self):
        self.calls = 0

    @method
    def add(self, a, b=0):
        self.calls += 1
        return a + b

    @method
    def boom(self):
        raise ValueError("nope")

    @method(raw=True)
    def echo(self, data):
        return data

    @method
    def nothing(self):
        return None

    @method(parallel=True)
    def slow(self, seconds):
        time.sleep(seconds)
        return "late"

    def not_exported(self):
        return 1


def test_wire_constants_and_registry_order():
    r = c.rpc
    assert (r.WIRE_VERSION, r.HEADER_SIZE, r.MAX_SLOT_COUNT) == (3, 16, 1 << 16)
    assert (r.EXC_BIT, r.ACK_BIT, r.REPLY_BIT, r.CHUNK_BIT, r.LAST_BIT) == (1 << 27, 1 << 28, 1 << 29, 1 << 30, 1 << 31)
    reg = MethodRegistry(Calc)
    assert [reg.by_tag[i].name for i in range(len(reg.by_tag))] == ["add", "boom", "echo", "nothing", "slow"]  # sorted names
    assert reg.by_name["echo"].raw and reg.by_name["slow"].parallel


@pytest.fixture()
def rpc_pair():
    ctrl = start_local_nanoctrl()
    w, d = PeerAgent(ctrl.url, alias="worker:0"), PeerAgent(ctrl.url, alias="driver:0")
    w._rpc_max_inflight = d._rpc_max_inflight = 4
    w._rpc_buffer_size = d._rpc_buffer_size = 4 << 20
    c1, c2 = d.connect_to("worker:0"), w.connect_to("driver:0")
    c1.wait(10)
    c2.wait(10)
    svc, stop = Calc(), threading.Event()
    t = threading.Thread(target=serve, args=(w, svc, "driver:0"), kwargs={"stop_event": stop}, daemon=True)
    t.start()
    yield proxy(d, "worker:0", Calc), svc, d
    stop.set()
    t.join(3)
    d.shutdown()
    w.shutdown()
    ctrl.stop()


def test_calls_results_and_remote_exception(rpc_pair):
    p, svc, _ = rpc_pair
    assert p.add(1, 2).wait(5) == 3 and p.add(5, b=6).wait(5) == 11 and p.nothing().wait(5) is None
    blob = bytes(range(256)) * 2000
    assert p.echo(blob).wait(5) == blob
    with pytest.raises(RemoteRpcError) as e:
        p.boom().wait(5)
    assert e.value.remote_type == "ValueError" and e.value.remote_message == "nope" and "Traceback" in e.value.remote_traceback
    assert p.add(1, 1).wait(5) == 2  # the session survives a remote exception
    assert not hasattr(p, "not_exported")
    with pytest.raises(RpcError, match="exceed the slot capacity"):
        p.echo(b"x" * (2 << 20))


def test_more_calls_than_slots_backpressure(rpc_pair):
    p, svc, _ = rpc_pair
    results = []

    def burst(k):
        results.extend(wait_all([p.add(k * 100 + i, 1) for i in range(3)], timeout=10))

    ts = [threading.Thread(target=burst, args=(k,)) for k in range(4)]  # 12 calls, 4 slots
    [t.start() for t in ts]
    [t.join(20) for t in ts]
    assert sorted(results) == sorted(k * 100 + i + 1 for k in range(4) for i in range(3))


def test_timeout_detaches_and_slot_is_reclaimed(rpc_pair):
    p, svc, d = rpc_pair
    with pytest.raises(RpcTimeoutError):
        p.slow(0.4).wait(0.05)
    time.sleep(0.6)  # the late reply arrives and only frees its slot
    assert [p.add(i, 0).wait(5) for i in range(8)] == list(range(8))  # all 4 slots are usable again
    sess = d._rpc_channels["worker:0"].session
    assert sess.requests_sent >= 9 and sess.replies_received >= 8


def test_close_fails_pending_calls(rpc_pair):
    p, svc, d = rpc_pair
    fut = p.slow(1.0)
    d._rpc_channels["worker:0"].session.close()
    with pytest.raises(RpcError):
        fut.wait(5)


def test_payload_sizes_around_the_slot_capacity():
    """Requests and replies up to exactly one slot's capacity pass; one byte more is refused on the side that would have
    sent it, with the limit in the message, and the session carries on."""
    from dlslime_b200.rpc import RemoteRpcError, RpcError

    class Blob:
        @method(raw=True)
        def echo(self, data):
            return data

        @method(raw=True)
        def grow(self, data):
            return bytes((i * 7) % 251 for i in range(int.from_bytes(data[:4], "little")))

    ctrl = start_local_nanoctrl()
    w, d = PeerAgent(ctrl.url, alias="worker:s"), PeerAgent(ctrl.url, alias="driver:s")
    for a in (w, d):
        a._rpc_max_inflight, a._rpc_buffer_size = 4, 64 << 10  # four slots of 16 KiB
    d.connect_to("worker:s").wait(10)
    w.connect_to("driver:s").wait(10)
    stop = threading.Event()
    t = threading.Thread(target=serve, args=(w, Blob(), "driver:s"), kwargs={"stop_event": stop}, daemon=True)
    t.start()
    try:
        p = proxy(d, "worker:s", Blob)
        cap = (16 << 10) - c.rpc.HEADER_SIZE
        for n in (0, 1, cap - 1, cap):
            payload = bytes((i * 3) % 256 for i in range(n))
            assert p.echo(payload).wait(10) == payload
            assert p.grow(n.to_bytes(4, "little")).wait(10) == bytes((i * 7) % 251 for i in range(n))
        for n in (cap + 1, 3 * cap):
            with pytest.raises(RpcError, match=str(cap)):
                p.echo(bytes(n)).wait(10)
            with pytest.raises(RemoteRpcError, match=str(cap)):
                p.grow(n.to_bytes(4, "little")).wait(10)
        assert p.echo(b"still in step").wait(10) == b"still in step"
        p.close()
    finally:
        stop.set()
        t.join(3)
        d.shutdown()
        w.shutdown()
        ctrl.stop()


def test_calls_from_many_threads_share_one_channel(rpc_pair):
    """Eight client threads on one proxy (four slots): bursts of serialised calls and parallel echoes, every reply goes
    to its own future and the serialised method ran exactly once per call."""
    p, svc, _ = rpc_pair
    errs = []

    def worker(t):
        try:
            for i in range(60):
                if i % 3 == 0:
                    futs = [p.add(i + k, t) for k in range(3)]
                    assert [f.wait(20) for f in futs] == [i + k + t for k in range(3)]
                else:
                    payload = bytes([t]) * (i % 50)
                    assert p.echo(payload).wait(20) == payload
        except Exception as e:  # noqa: BLE001
            errs.append((t, repr(e)))

    ths = [threading.Thread(target=worker, args=(t,)) for t in range(8)]
    [t.start() for t in ths]
    [t.join(120) for t in ths]
    assert not errs and not any(t.is_alive() for t in ths)
    assert svc.calls == 8 * 20 * 3
