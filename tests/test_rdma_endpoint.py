"""RDMA endpoint, context, channel logic and worker on the software loopback fabric (no NIC needed).

Covers what the reference's RDMA tests need hardware for (tests/python/test_rdma_*.py in the reference):
one-sided read / write with striping over queue pairs, write-with-immediate ordering over lanes,
immediate events that arrive before / after imm_recv, rendezvous send / recv (ordering, overflow), credit
back-pressure with batches larger than the send queue, failure statuses (bad remote key, injected
completion error), cancel_all and shutdown.
"""
import ctypes
import os
import subprocess
import sys
import textwrap

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_child(body: str, env_extra=None, timeout=120):
    env = dict(os.environ, SLIME_RDMA_PROVIDER="loopback", PYTHONPATH=REPO)
    env.update(env_extra or {})
    prelude = textwrap.dedent("""
        import ctypes, os, sys, threading, time
        from dlslime_b200 import _slime_c as C

        def buf(n, fill=None):
            b = (ctypes.c_ubyte * n)()
            if fill is not None:
                ctypes.memset(b, fill, n)
            return b

        def pair(num_qp=2, dev_a="rdma_lo0", dev_b="rdma_lo0"):
            a = C.RDMAEndpoint(dev_a, 1, "", num_qp)
            b = C.RDMAEndpoint(dev_b, 1, "", num_qp)
            return a, b

        def link(a, b):
            ia, ib = a.endpoint_info(), b.endpoint_info()
            assert a.connect(ib) == 0 and b.connect(ia) == 0
    """)
    r = subprocess.run([sys.executable, "-c", prelude + textwrap.dedent(body)], env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, f"child failed\nstdout:\n{r.stdout}\nstderr:\n{r.stderr}"
    return r.stdout


def test_provider_selection_and_context():
    out = run_child("""
        assert C._BUILD_RDMA
        name, why = C.rdma_provider()
        assert name == "loopback", (name, why)
        assert C.rdma_devices() == ["rdma_lo0", "rdma_lo1", "rdma_lo2"]
        ctx = C.RDMAContext.acquire("rdma_lo0", 1, "RoCE")
        assert ctx.link_type() == "RoCE" and ctx.gid_index() == 1 and ctx.mtu() == 5
        ib = C.RDMAContext.acquire("rdma_lo1", 1, "IB")
        assert ib.link_type() == "IB" and ib.lid() == 7
        try:
            C.RDMAContext.acquire("rdma_lo1", 1, "RoCE")   # cached under the same key: asks again with another link type
        except RuntimeError:
            pass
        # an unknown device falls back to the first one
        fb = C.RDMAContext.acquire("mlx5_nope", 1, "")
        assert fb.device_name() == "rdma_lo0"
        # link-type mismatch on a fresh key is refused
        try:
            C.RDMAContext.acquire("rdma_lo0", 2, "IB")
            raise SystemExit("port 2 is not active; must fail")
        except RuntimeError as e:
            assert "not active" in str(e)
        print("ok")
    """)
    assert "ok" in out


def test_without_provider_reports_reason():
    out = run_child("""
        name, why = C.rdma_provider()
        print(name, "|", why)
        try:
            C.RDMAEndpoint("", 1, "", 1)
            print("created")
        except RuntimeError as e:
            print("refused:", e)
    """, env_extra={"SLIME_RDMA_PROVIDER": "ibverbs"})
    # this host has no libibverbs / no NIC: the endpoint refuses with the reason; with a NIC it would be created
    assert "refused: no RDMA provider" in out or "created" in out


def test_one_sided_read_write_striped():
    out = run_child("""
        a, b = pair(num_qp=4)
        n = 1 << 20
        src = buf(n); dst = buf(n); back = buf(n)
        for i in range(n):
            pass
        ctypes.memmove(src, bytes((i * 7 + 3) & 0xff for i in range(n)), n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        a.register_memory_region("back", ctypes.addressof(back), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        assert ha >= 0 and hb >= 0
        # (local, remote, remote_off, local_off, len): one big striped piece, small pieces round-robin, odd offsets
        f = a.write([(ha, hb, 0, 0, 512 << 10), (ha, hb, (512 << 10) + 5, (512 << 10) + 5, 1000), (ha, hb, 700000, 700000, 3)])
        assert f.wait(5000) == 0
        assert bytes(dst[:512 << 10]) == bytes(src[:512 << 10])
        assert bytes(dst[(512 << 10) + 5:(512 << 10) + 1005]) == bytes(src[(512 << 10) + 5:(512 << 10) + 1005])
        assert bytes(dst[700000:700003]) == bytes(src[700000:700003]) and dst[700003] == 0
        # 4 stripes + 2 unstriped pieces
        assert a.posted_wrs() == 6, a.posted_wrs()
        hback = a.get_mr_handle("back")
        f = a.read([(hback, hb, 0, 0, 512 << 10)])
        assert f.wait(5000) == 0 and bytes(back[:512 << 10]) == bytes(src[:512 << 10])
        # an empty batch completes at once
        assert a.write([]).wait(1000) == 0
        a.shutdown(); b.shutdown()
        print("ok")
    """)
    assert "ok" in out


def test_write_with_imm_all_lanes_and_event_queue():
    out = run_child("""
        a, b = pair(num_qp=3)
        n = 300000
        src = buf(n, 0x5a); dst = buf(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        # events that arrive before anyone asks are queued in order
        for k in range(5):
            assert a.write_with_imm([(ha, hb, k * 10, k * 10, 10)], 100 + k).wait(5000) == 0
        got = []
        for k in range(5):
            f = b.imm_recv()
            assert f.wait(5000) == 0
            got.append(f.imm_data())
        assert got == [100, 101, 102, 103, 104], got
        # a waiter that is posted first is completed by the next event; a striped payload has landed by then
        f = b.imm_recv()
        assert f.wait(50) == 402          # TIME_OUT, still pending
        assert a.write_with_imm([(ha, hb, 0, 0, n)], 7).wait(5000) == 0
        assert f.wait(5000) == 0 and f.imm_data() == 7
        assert bytes(dst) == bytes(src)
        # every lane carried exactly one immediate per operation: 6 ops x 3 lanes signaled at least that many
        assert a.signaled_wrs() >= 18
        a.shutdown(); b.shutdown()
        print("ok")
    """)
    assert "ok" in out


def test_send_recv_rendezvous_order_and_overflow():
    out = run_child("""
        a, b = pair(num_qp=2)
        link(a, b)
        msgs = [bytes([k]) * (1000 + k * 70000) for k in range(4)]
        sbufs = [ctypes.create_string_buffer(m, len(m)) for m in msgs]
        rbufs = [ctypes.create_string_buffer(len(m)) for m in msgs]
        # receives first on b, sends on a; then the other way round for the last two
        rf = [b.recv((ctypes.addressof(rbufs[k]), 0, len(msgs[k]))) for k in range(2)]
        sf = [a.send((ctypes.addressof(sbufs[k]), 0, len(msgs[k]))) for k in range(4)]
        rf += [b.recv((ctypes.addressof(rbufs[k]), 0, len(msgs[k]))) for k in range(2, 4)]
        for f in sf + rf:
            assert f.wait(5000) == 0
        for k in range(4):
            assert rbufs[k].raw == msgs[k], k
        # a send larger than the posted receive buffer: both sides learn it (400), nothing past the buffer is written
        small = ctypes.create_string_buffer(64 + 8)
        big = ctypes.create_string_buffer(b"x" * 128, 128)
        r = b.recv((ctypes.addressof(small), 0, 64))
        s = a.send((ctypes.addressof(big), 0, 128))
        assert s.wait(5000) == 400 and r.wait(5000) == 400
        assert small.raw[:64] == b"x" * 64 and small.raw[64:] == bytes(8)
        a.shutdown(); b.shutdown()
        print("ok")
    """)
    assert "ok" in out


def test_credit_backpressure_and_signal_interval():
    out = run_child("""
        a, b = pair(num_qp=1)
        n = 64 * 1000
        src = buf(n, 1); dst = buf(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        # 1000 work requests through a send queue of 64 credits
        f = a.write([(ha, hb, i * 64, i * 64, 64) for i in range(1000)])
        assert f.wait(10000) == 0
        assert bytes(dst) == bytes(src)
        assert a.posted_wrs() == 1000
        assert a.signaled_wrs() == 32, a.signaled_wrs()      # every 32nd (31) + the last one
        assert a.credit_stalls() > 0
        a.shutdown(); b.shutdown()
        print("ok")
    """, env_extra={"SLIME_MAX_SEND_WR": "64"})
    assert "ok" in out


def test_failures_cancel_and_shutdown():
    out = run_child("""
        a, b = pair(num_qp=2)
        n = 4096
        src = buf(n, 9); dst = buf(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        # out-of-range assignment is refused before anything is posted
        f = a.write([(ha, hb, n - 10, 0, 100)])
        try:
            f.wait(1000); raise SystemExit("must throw")
        except RuntimeError as e:
            assert "403" in str(e)
        # the peer drops its region: the stale remote key fails the transfer with FAILED, the future throws
        b.unregister_memory_region("dst")
        f = a.write([(ha, hb, 0, 0, 100)])
        try:
            f.wait(5000); raise SystemExit("must throw")
        except RuntimeError as e:
            assert "403" in str(e)
        # pending immediate waiters are failed by cancel_all
        w = b.imm_recv()
        b.cancel_all()
        assert w.wait(1000) == 403
        a.shutdown(); a.shutdown(); b.shutdown()
        # after shutdown every call fails fast
        try:
            a.write([(ha, hb, 0, 0, 1)]).wait(1000); raise SystemExit("must throw")
        except RuntimeError:
            pass
        snap = C.obs_snapshot()
        print("ok")
    """, env_extra={"DLSLIME_OBS": "1"})
    assert "ok" in out


def test_injected_completion_error_and_recovery_on_new_endpoint():
    out = run_child("""
        a, b = pair(num_qp=1)
        n = 1 << 16
        src = buf(n, 3); dst = buf(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        C.rdma_loopback_inject_error(0, 12, 1)     # next WRITE completes with retry-exceeded
        f = a.write([(ha, hb, i * 64, i * 64, 64) for i in range(100)])
        try:
            f.wait(5000); raise SystemExit("must throw")
        except RuntimeError as e:
            assert "403" in str(e)
        a.shutdown(); b.shutdown()
        # a fresh pair works again
        a2, b2 = pair(num_qp=1)
        a2.register_memory_region("src", ctypes.addressof(src), 0, n)
        b2.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a2, b2)
        assert a2.write([(a2.get_mr_handle("src"), a2.get_remote_mr_handle("dst"), 0, 0, n)]).wait(5000) == 0
        assert bytes(dst) == bytes(src)
        a2.shutdown(); b2.shutdown()
        print("ok")
    """)
    assert "ok" in out


def test_peer_agent_over_rdma_links():
    """Two agents in one process, each on a RoCE device of its own: handshake through the control plane, named
    I/O with keys published per resource, write-with-immediate, a region registered after the link came up."""
    out = run_child("""
        from dlslime_b200.nanoctrl import start_local_nanoctrl
        from dlslime_b200.peer_agent import PeerAgent
        ctrl = start_local_nanoctrl()
        a = PeerAgent(ctrl.url, alias="A", scope="r", device="rdma_lo0", link_type="RoCE")
        b = PeerAgent(ctrl.url, alias="B", scope="r", device="rdma_lo2", link_type="RoCE")
        try:
            n = 1 << 18
            ba = ctypes.create_string_buffer(bytes((i * 3 + 1) & 0xff for i in range(n)), n)
            bb = ctypes.create_string_buffer(n)
            a.register_memory_region("kv", ctypes.addressof(ba), 0, n)
            b.register_memory_region("kv", ctypes.addressof(bb), 0, n)
            conn = a.connect_to("B", local_device="rdma_lo0", peer_device="rdma_lo2").wait(10)
            assert conn.is_connected() and (conn.local_nic, conn.remote_nic) == ("rdma_lo0", "rdma_lo2"), conn.conn_id
            assert a.write("B", [("kv", 0, 4096, 200000)]).wait(10) == 0
            assert bb.raw[4096:204096] == ba.raw[:200000]
            assert b.query_connection("A").wait(5).is_connected()
            assert b.read("A", ("kv", "kv", 0, 7, 100)).wait(10) == 0 and bb.raw[:100] == ba.raw[7:107]
            assert a.write_with_imm("B", [("kv", 0, 0, 16)], imm_data=77).wait(10) == 0
            f = b.imm_recv("A")
            assert f.wait(10) == 0 and f.imm_data() == 77
            late = ctypes.create_string_buffer(b"z" * 512, 512)
            b.register_memory_region("late", ctypes.addressof(late), 0, 512)
            got = ctypes.create_string_buffer(512)
            a.register_memory_region("got", ctypes.addressof(got), 0, 512)
            assert a.read("B", ("got", "late", 0, 0, 512)).wait(10) == 0 and got.raw == b"z" * 512
        finally:
            a.shutdown(); b.shutdown(); ctrl.stop()
        print("ok")
    """)
    assert "ok" in out


def test_obs_counts_each_operation_once_with_four_queue_pairs():
    """Accounting is per user operation, not per queue pair or work request (the reference pins this in
    tests/python/test_obs_multi_qp.py): bytes completed equal bytes submitted, nothing stays pending."""
    out = run_child("""
        a, b = pair(num_qp=4)
        n = 8 << 20
        src = buf(n, 1); dst = buf(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        link(a, b)
        ha, hb = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        total = 0   # a fresh process: every counter starts at zero
        for k in range(10):
            assert a.write([(ha, hb, 0, 0, 1 << 20), (ha, hb, 1 << 20, 1 << 20, 4096)]).wait(5000) == 0
            total += (1 << 20) + 4096
        assert a.read([(ha, hb, 0, 0, 2 << 20)]).wait(5000) == 0
        snap = C.obs_snapshot()
        nic = [x for x in snap["nics"] if x["nic"] == "rdma_lo0"][0]
        w, r = nic["by_op"]["write"], nic["by_op"]["read"]
        assert w["batch"] == 10 and w["assign"] == 20 and w["errors"] == 0 and w["pending"] == 0, w
        assert w["completed_bytes"] == total and w["submitted_bytes"] == total, w
        assert r["batch"] == 1 and r["completed_bytes"] == 2 << 20, r
        assert snap["summary"]["pending_ops"] == 0 and nic["pending_ops"] == 0, snap["summary"]
        assert w["post_wr"] == 10 * 5 and w["post_bytes"] == total, w      # 4 stripes + 1 small piece per write, counted apart
        a.shutdown(); b.shutdown()
        print("ok")
    """, env_extra={"DLSLIME_OBS": "1"})
    assert "ok" in out


def test_slimerpc_over_rdma_links():
    """SlimeRPC (slot mailbox written with write_with_imm, immediates as slot ids) between two agents connected over
    RoCE-typed links with two queue pairs: calls, a burst of calls in flight, a large reply that is chunked, a remote exception."""
    out = run_child("""
        from dlslime_b200.nanoctrl import start_local_nanoctrl
        from dlslime_b200.peer_agent import PeerAgent
        from dlslime_b200.rpc import method, proxy, serve
        from dlslime_b200.rpc.errors import RemoteRpcError

        class Svc:
            @method
            def add(self, a, b):
                return a + b
            @method
            def blob(self, n):
                return bytes(i % 251 for i in range(n))
            @method
            def boom(self):
                raise ValueError("no such block")

        ctrl = start_local_nanoctrl()
        w = PeerAgent(ctrl.url, alias="w", scope="rr", device="rdma_lo0", link_type="RoCE")
        d = PeerAgent(ctrl.url, alias="d", scope="rr", device="rdma_lo2", link_type="RoCE")
        stop = threading.Event()
        try:
            d.connect_to("w", local_device="rdma_lo2", peer_device="rdma_lo0", qp_num=2).wait(10)
            w.connect_to("d", local_device="rdma_lo0", peer_device="rdma_lo2", qp_num=2).wait(10)
            threading.Thread(target=serve, args=(w, Svc(), "d"), kwargs={"stop_event": stop}, daemon=True).start()
            p = proxy(d, "w", Svc)
            assert p.add(2, 3).wait(10) == 5
            futs = [p.add(i, i) for i in range(32)]
            assert [f.wait(10) for f in futs] == [2 * i for i in range(32)]
            big = p.blob(600_000).wait(20)
            assert len(big) == 600_000 and big[:5] == bytes([0, 1, 2, 3, 4]) and big[-1] == (599_999 % 251)
            try:
                p.boom().wait(10); raise SystemExit("must raise")
            except RemoteRpcError as e:
                assert "no such block" in str(e)
            p.close()
        finally:
            stop.set(); d.shutdown(); w.shutdown(); ctrl.stop()
        print("ok")
    """, timeout=180)
    assert "ok" in out


def test_random_batches_match_a_model_and_bad_batches_fail_cleanly():
    """Seeded random batches of reads and writes (zero lengths, stripes over four queue pairs, pieces that end exactly at
    the region's end) against two byte arrays; a batch with a piece past its region fails, and the endpoint keeps working."""
    out = run_child("""
        import random
        rnd = random.Random(11)
        n = 1 << 18
        a, b = pair(num_qp=4)
        la, rb = buf(n), buf(n)
        local, remote = bytearray(rnd.randbytes(n)), bytearray(rnd.randbytes(n))
        ctypes.memmove(la, bytes(local), n); ctypes.memmove(rb, bytes(remote), n)
        # endpoints on one device share that device's registry, so the two regions need different names in one process
        a.register_memory_region("near", ctypes.addressof(la), 0, n)
        b.register_memory_region("far", ctypes.addressof(rb), 0, n)
        link(a, b)
        lh, rh = a.get_mr_handle("near"), a.get_remote_mr_handle("far")
        sizes = [0, 1, 7, 64, 1000, 4096, 65536, 100_000, n]
        bad_seen = 0
        for step in range(150):
            op = rnd.choice(["read", "write"])
            pieces = []
            for _ in range(rnd.randint(1, 6)):
                ln = rnd.choice(sizes)
                if rnd.random() < 0.1:   # sometimes out of range on one side
                    ro, lo = rnd.randint(0, n), rnd.randint(0, n)
                else:
                    ro, lo = rnd.randint(0, n - ln), rnd.randint(0, n - ln)
                pieces.append((ro, lo, ln))
            # destinations of one batch must not overlap (stripes of different pieces run concurrently)
            dst = sorted(((lo, lo + ln) if op == "read" else (ro, ro + ln)) for ro, lo, ln in pieces if ln)
            if any(x[1] > y[0] for x, y in zip(dst, dst[1:])):
                continue
            ok = all(ro + ln <= n and lo + ln <= n for ro, lo, ln in pieces)
            fut = getattr(a, op)([(lh, rh, ro, lo, ln) for ro, lo, ln in pieces])
            if not ok:
                bad_seen += 1
                try:
                    st = fut.wait(5000)
                    assert st != 0, (step, op, pieces)
                except RuntimeError:
                    pass
                # whatever part of a failed batch landed, the endpoints must stay usable; resynchronise the model
                local[:] = bytes(la); remote[:] = bytes(rb)
                if not a.connected():
                    break
                continue
            assert fut.wait(5000) == 0, (step, op, pieces)
            for ro, lo, ln in pieces:
                if op == "write":
                    remote[ro:ro + ln] = local[lo:lo + ln]
                else:
                    local[lo:lo + ln] = remote[ro:ro + ln]
            assert bytes(la) == bytes(local) and bytes(rb) == bytes(remote), (step, op, pieces)
        assert a.write([(lh, rh, 0, 0, 16)]).wait(5000) == 0
        a.shutdown(); b.shutdown()
        print("ok", bad_seen)
    """, timeout=240)
    assert "ok" in out


def test_reference_style_pool_worker_and_constructor_forms():
    """Code written against the reference's classes runs unchanged: ``RDMAMemoryPool(context)``,
    ``RDMAWorker(socket_id, id)`` with start / add_endpoint / stop, and the three ``RDMAEndpoint`` constructors
    (pool, context, device name), each with an optional worker (dlslime/csrc/python/bind.cpp:163-204,272 in the
    reference)."""
    out = run_child("""
        ctx = C.RDMAContext.acquire("rdma_lo0", 1, "RoCE")
        pool = C.RDMAMemoryPool(ctx)
        worker = C.RDMAWorker(0, 0)
        by_name = C.RDMAWorker("rdma_lo0", 1)
        assert not worker.running()
        worker.start()
        assert worker.running()
        n = 1 << 20
        src, dst = buf(n, 0x5a), buf(n, 0)
        hs = pool.register_memory_region(ctypes.addressof(src), n, "src")
        hd = pool.register_memory_region(ctypes.addressof(dst), n, "dst")
        assert pool.get_handle("src") == hs and set(pool.mr_info()) >= {"src", "dst"}
        a = C.RDMAEndpoint(pool, 2, worker)                     # form 1: pool, num_qp, worker
        b = C.RDMAEndpoint(ctx, num_qp=2)                       # form 2: context (shared per-node worker)
        c = C.RDMAEndpoint("rdma_lo0", 1, "RoCE", 2, by_name)   # form 3: device name ... worker (not started yet)
        assert a.get_pool().get_handle("dst") == hd             # one registry per device: every view sees the regions
        link(a, b)
        for name, info in b.endpoint_info()["mr_info"].items():
            a.register_remote_memory_region(name, info)
        rh = a.get_remote_mr_handle("dst")
        assert a.write([(hs, rh, 0, 0, n)]).wait(10) == 0
        assert bytes(dst[:16]) == bytes([0x5a]) * 16 and dst[n - 1] == 0x5a
        loops = worker.stats()["loops"]
        assert loops > 0
        # stopping the caller's worker hands its endpoints back to the shared one: traffic goes on
        worker.stop()
        assert not worker.running()
        ctypes.memset(src, 0x33, n)
        assert a.write([(hs, rh, 4096, 4096, 8192)]).wait(10) == 0
        assert dst[4096] == 0x33 and dst[4095] == 0x5a
        # a worker that is started after its endpoint was added takes the endpoint over
        by_name.start(); assert by_name.running()
        by_name.stop()
        assert pool.unregister_memory_region("src") == 0
        for ep in (a, b, c):
            ep.shutdown()
        print("ok")
    """)
    assert "ok" in out
