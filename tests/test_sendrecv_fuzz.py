"""Two-sided send / recv under seeded random interleavings, on the TCP endpoint and on the RDMA engine over the software
fabric: the i-th send meets the i-th receive whatever the order of issue, payloads arrive byte for byte, a buffer that is
too small is reported to the receiver (status 400) with the part that fits."""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import ctypes, os, sys, random
from dlslime_b200 import _slime_c as C
kind = sys.argv[1]
if kind == "rdma":
    a, b = C.RDMAEndpoint("rdma_lo0", 1, "", 2), C.RDMAEndpoint("rdma_lo0", 1, "", 2)
else:
    a, b = C.TcpEndpoint(), C.TcpEndpoint()
ia, ib = a.endpoint_info(), b.endpoint_info()
assert a.connect(ib) == 0 and b.connect(ia) == 0
rnd = random.Random(int(sys.argv[2]) if len(sys.argv) > 2 else 1)
CAP = 1 << 17
for rounds in range(60):
    k = rnd.randint(1, 6)
    msgs = [bytes(rnd.randrange(256) for _ in range(8)) * rnd.choice([0, 1, 8, 500, 4000, CAP // 8]) for _ in range(k)]
    caps = [len(m) + rnd.choice([0, 0, 16, -4 if len(m) >= 8 else 0]) for m in msgs]  # sometimes a buffer that is too small
    sb = [ctypes.create_string_buffer(m, max(len(m), 1)) for m in msgs]
    rb = [ctypes.create_string_buffer(max(c, 1)) for c in caps]
    order = ["s"] * k + ["r"] * k
    rnd.shuffle(order)
    si = ri = 0
    sf, rf = [], []
    for o in order:  # sends and receives are issued in their own order; the i-th send meets the i-th recv
        if o == "s":
            sf.append(a.send((ctypes.addressof(sb[si]), 0, len(msgs[si])))); si += 1
        else:
            rf.append(b.recv((ctypes.addressof(rb[ri]), 0, caps[ri]))); ri += 1
    for i in range(k):
        ss, rs = sf[i].wait(10_000), rf[i].wait(10_000)
        if caps[i] >= len(msgs[i]):
            assert (ss, rs) == (0, 0), (rounds, i, ss, rs, len(msgs[i]), caps[i])
            assert rb[i].raw[:len(msgs[i])] == msgs[i], (rounds, i)
        else:
            assert rs == 400, (rounds, i, ss, rs, len(msgs[i]), caps[i])   # the receiver learns that its buffer was too small
            assert rb[i].raw[:caps[i]] == msgs[i][:caps[i]]
print("ok", kind)
a.shutdown(); b.shutdown()
'''


@pytest.mark.parametrize("transport,seed", [("tcp", 1), ("tcp", 2), ("rdma", 1), ("rdma", 2)])
def test_send_recv_random_interleavings(transport, seed):
    env = dict(os.environ, PYTHONPATH=REPO, SLIME_RDMA_PROVIDER="loopback")
    r = subprocess.run([sys.executable, "-c", WORKER, transport, str(seed)], env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and f"ok {transport}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


IMM_WORKER = r'''
import ctypes, sys, random, threading
from dlslime_b200 import _slime_c as C
kind = sys.argv[1]; seed = int(sys.argv[2])
if kind == "rdma":
    a, b = C.RDMAEndpoint("rdma_lo0", 1, "", 4), C.RDMAEndpoint("rdma_lo0", 1, "", 4)
else:
    a, b = C.TcpEndpoint("127.0.0.1", 0, 2), C.TcpEndpoint("127.0.0.1", 0, 2)
n = 1 << 20
src, dst = ctypes.create_string_buffer(n), ctypes.create_string_buffer(n)
a.register_memory_region("near", ctypes.addressof(src), 0, n)
b.register_memory_region("far", ctypes.addressof(dst), 0, n)
ia, ib = a.endpoint_info(), b.endpoint_info()
assert a.connect(ib) == 0 and b.connect(ia) == 0
if kind != "rdma":
    a.register_remote_memory_region("far", ib["mr_info"]["far"])
lh, rh = a.get_mr_handle("near"), a.get_remote_mr_handle("far")
rnd = random.Random(seed)
K = 120
plan = []
for k in range(K):
    ln = rnd.choice([0, 1, 64, 4096, 8192])
    off = k * 8192   # disjoint slots: a later write never touches what an earlier event is checked against
    plan.append((off, ln, k + 1000))
events = []
def receiver():
    for k in range(K):
        if rnd.random() < 0.3:
            pass
        f = b.imm_recv()
        assert f.wait(20_000) == 0
        imm = f.imm_data()
        off, ln, want = plan[k]
        # the data of the k-th write is in place when its immediate is delivered
        ok = dst.raw[off:off + ln] == bytes([(k * 7 + 1) % 256]) * ln
        events.append((imm, want, ok))
t = threading.Thread(target=receiver); t.start()
futs = []
for k, (off, ln, imm) in enumerate(plan):
    ctypes.memset(ctypes.addressof(src) + off, (k * 7 + 1) % 256, ln)
    f = a.write_with_imm([(lh, rh, off, off, ln)], imm)
    futs.append(f)
for f in futs:
    assert f.wait(20_000) == 0
t.join(60)
assert not t.is_alive()
bad = [(i, e) for i, e in enumerate(events) if e[0] != e[1] or not e[2]]
assert not bad, bad[:5]
print("ok", kind, len(events))
a.shutdown(); b.shutdown()
'''


@pytest.mark.parametrize("transport,seed", [("tcp", 1), ("rdma", 1), ("rdma", 2)])
def test_immediates_arrive_in_order_with_their_data(transport, seed):
    """120 writes with immediate data in flight at once (random sizes, striped over four queue pairs on the RDMA engine):
    the k-th event carries the k-th immediate, and the bytes of that write are in place when it is delivered."""
    env = dict(os.environ, PYTHONPATH=REPO, SLIME_RDMA_PROVIDER="loopback", SLIME_STRIPE_MIN_BYTES="1024")
    r = subprocess.run([sys.executable, "-c", IMM_WORKER, transport, str(seed)], env=env, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and f"ok {transport}" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
