"""TCP endpoint: both endpoints live in one process (the reference tests its RDMA endpoint the same
way, through NIC loopback). Byte-exact windows, immediate-data ordering, send/recv matching, shutdown
that wakes blocked waiters, and host-side fault injection."""
import ctypes
import random
import threading
import time

import pytest

from dlslime_b200 import _slime_c as c

N = 4 << 20


def _buf(seed=None):
    b = ctypes.create_string_buffer(N)
    if seed is not None:
        rnd = random.Random(seed)
        b.raw = bytes(rnd.getrandbits(8) for _ in range(4096)) * (N // 4096)
    return b


@pytest.fixture()
def pair():
    a, b = c.TcpEndpoint(), c.TcpEndpoint()
    ba, bb = _buf(1), _buf(2)
    a.register_memory_region("buf", ctypes.addressof(ba), 0, N)
    b.register_memory_region("buf", ctypes.addressof(bb), 0, N)
    a.connect(b.endpoint_info())
    b.connect(a.endpoint_info())
    yield a, b, ba, bb
    a.shutdown()
    b.shutdown()


def test_endpoint_info_shape(pair):
    a, *_ = pair
    info = a.endpoint_info()
    assert info["kind"] == "tcp" and info["port"] == a.port() and set(info["mr_info"]["buf"]) >= {"handle", "addr", "rkey", "length"}


def test_many_concurrent_windows_are_byte_exact(pair):
    a, b, ba, bb = pair
    rnd = random.Random(0)
    ops, expect_b, expect_a = [], bytearray(bb.raw), bytearray(ba.raw)
    # disjoint 4 KiB windows: writes go to even windows of B, reads land in odd windows of A
    for i in range(256):
        n = rnd.randrange(1, 4096)
        src = rnd.randrange(0, N - 4096)
        if i % 2 == 0:
            dst = (2 * i) * 4096
            ops.append(a.write([(0, 0, dst, src, n)]))
            expect_b[dst:dst + n] = ba.raw[src:src + n]
        else:
            dst = (2 * i + 1) * 4096
            ops.append(a.read([(0, 0, src, dst, n)]))
            expect_a[dst:dst + n] = bb.raw[src:src + n]
    assert all(f.wait(10) == 0 for f in ops)
    assert bb.raw == bytes(expect_b) and ba.raw == bytes(expect_a)


def test_batched_assignment_and_bounds(pair):
    a, b, ba, bb = pair
    f = a.write([(0, 0, 100 * i, 200 * i, 50) for i in range(100)])
    assert f.wait(10) == 0
    assert all(bb.raw[100 * i:100 * i + 50] == ba.raw[200 * i:200 * i + 50] for i in range(100))
    bad = a.write([(0, 0, N - 10, 0, 100)])  # runs past the remote region
    with pytest.raises(RuntimeError, match="status 403"):
        bad.wait(10)
    bad = a.read([(0, 5, 0, 0, 16)])  # unknown remote handle
    with pytest.raises(RuntimeError):
        bad.wait(10)
    assert a.write([(0, 0, 0, 0, 16)]).wait(10) == 0  # the connection is still usable


@pytest.mark.parametrize("order", ["recv_first", "send_first", "interleaved"])
def test_imm_values_arrive_once_each(pair, order):
    a, b, *_ = pair
    k = 64
    futs = []
    if order == "recv_first":
        futs = [b.imm_recv() for _ in range(k)]
    for i in range(k):
        assert a.write_with_imm([(0, 0, i * 64, i * 64, 64)], 1000 + i).wait(10) == 0
        if order == "interleaved":
            futs.append(b.imm_recv())
    if order == "send_first":
        futs = [b.imm_recv() for _ in range(k)]
    assert all(f.wait(10) == 0 for f in futs)
    assert sorted(f.imm_data() for f in futs) == [1000 + i for i in range(k)]
    assert futs[0].time_trace_enabled() and futs[0].time_trace_end_ns() >= futs[0].time_trace_start_ns()


def test_send_recv_pairs_in_order(pair):
    a, b, ba, bb = pair
    recvs = [b.recv((ctypes.addressof(bb), i * 1024, 1024)) for i in range(8)]  # posted first
    sends = [a.send((ctypes.addressof(ba), 7000 + i * 1024, 1024)) for i in range(8)]
    assert all(f.wait(10) == 0 for f in sends + recvs)
    assert all(bb.raw[i * 1024:(i + 1) * 1024] == ba.raw[7000 + i * 1024:7000 + (i + 1) * 1024] for i in range(8))
    s = a.send((ctypes.addressof(ba), 0, 333))  # unexpected message is buffered until a recv is posted
    assert s.wait(10) == 0
    r = b.recv((ctypes.addressof(bb), 500000, 1024))
    assert r.wait(10) == 0 and bb.raw[500000:500333] == ba.raw[:333]


def test_shutdown_wakes_blocked_waiters_with_failed_status(pair):
    a, b, *_ = pair
    results = []
    waiters = [b.imm_recv() for _ in range(8)]
    ts = [threading.Thread(target=lambda f=f: results.append(f.wait(30))) for f in waiters]
    [t.start() for t in ts]
    time.sleep(0.05)
    t0 = time.monotonic()
    b.shutdown()
    [t.join(5) for t in ts]
    assert results == [403] * 8 and time.monotonic() - t0 < 5
    b.shutdown()  # idempotent
    assert b.imm_recv().wait(1) == 403


def test_peer_exit_fails_in_flight_operations(pair):
    a, b, *_ = pair
    b.shutdown()
    time.sleep(0.05)
    f = a.write([(0, 0, 0, 0, 1024)])
    with pytest.raises(RuntimeError):
        f.wait(5)


def test_injected_faults(pair):
    a, b, *_ = pair
    b.inject_fault("fail_write", 1)
    with pytest.raises(RuntimeError, match="403"):
        a.write([(0, 0, 0, 0, 64)]).wait(5)
    assert a.write([(0, 0, 0, 0, 64)]).wait(5) == 0
    a.inject_fault("drop_ack", 1)
    lost = a.write([(0, 0, 0, 0, 64)])
    assert lost.wait(0.2) == 402  # a lost acknowledgement shows up as a timeout, not a hang
    a.inject_fault("reset", 1)
    with pytest.raises(RuntimeError):
        a.write([(0, 0, 0, 0, 64)]).wait(5)


def test_oversized_message_closes_the_connection_instead_of_the_process():
    """The length of a two-sided message comes from the peer. Above SLIME_TCP_MAX_MESSAGE_BYTES the receiving side
    closes the connection (the sender's operation fails) and nothing is allocated for it; the process lives on."""
    import os
    import subprocess
    import sys
    import textwrap

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    body = textwrap.dedent("""
        import ctypes
        from dlslime_b200 import _slime_c as c
        n = 1 << 16
        ba, bb = ctypes.create_string_buffer(n), ctypes.create_string_buffer(n)
        a, b = c.TcpEndpoint(), c.TcpEndpoint()
        a.register_memory_region("buf", ctypes.addressof(ba), 0, n)
        b.register_memory_region("buf", ctypes.addressof(bb), 0, n)
        a.connect(b.endpoint_info()); b.connect(a.endpoint_info())
        ok = a.send((ctypes.addressof(ba), 0, 512))
        r = b.recv((ctypes.addressof(bb), 0, 1024))
        assert ok.wait(5) == 0 and r.wait(5) == 0
        big = a.send((ctypes.addressof(ba), 0, 4096))      # above the 1 KiB limit set below
        st = big.wait(5)
        assert st in (402, 403), st
        a.shutdown(); b.shutdown()
        print("alive")
    """)
    env = dict(os.environ, PYTHONPATH=repo, SLIME_TCP_MAX_MESSAGE_BYTES="1024")
    r = subprocess.run([sys.executable, "-c", body], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "alive" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_operations_of_one_thread_leave_in_submission_order_whatever_their_size(pair):
    """Small operations are posted by the submitting thread when nothing is queued, large ones by the sender thread. A
    stream of alternating 1 MiB and 8-byte writes with immediates, submitted without waiting, must still reach the peer in
    submission order: the immediates arrive as 0, 1, 2, ... and the word that every small write targets ends up holding
    the last small write's value."""
    a, b, ba, bb = pair
    k = 64
    word = 3 << 20  # offset of the 8-byte word in both buffers
    futs = []
    for i in range(k):
        if i % 2 == 0:
            futs.append(a.write_with_imm([(0, 0, 0, 0, 1 << 20)], i))
        else:
            ctypes.memmove(ctypes.addressof(ba) + (1 << 21) + 8 * i, i.to_bytes(8, "little"), 8)  # a distinct source per write
            futs.append(a.write_with_imm([(0, 0, word, (1 << 21) + 8 * i, 8)], i))
    assert all(f.wait(20) == 0 for f in futs)
    got = []
    for _ in range(k):
        r = b.imm_recv()
        assert r.wait(10) == 0
        got.append(r.imm_data())
    assert got == list(range(k))
    assert int.from_bytes(bb.raw[word:word + 8], "little") == k - 1
