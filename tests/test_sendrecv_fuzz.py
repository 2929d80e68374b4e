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
