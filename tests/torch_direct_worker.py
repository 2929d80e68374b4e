"""Worker of test_torch_backend_direct.py: the rendezvous protocol of the GPU-direct path (the receiver exports its
buffer, the sender copies into it) run on host tensors with shared memory in place of CUDA IPC."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import dlslime_b200.torch_backend  # noqa: F401,E402  (registers the backend)


def main():
    dist.init_process_group("dlslime")
    rank = dist.get_rank()
    peer = 1 - rank
    pg = dist.distributed_c10d._get_default_group()
    assert type(pg).__name__ == "DirectGroup", type(pg)  # a Python process group is used as the group itself
    # ordered pairs, sizes from one element to a few MB, including an empty tensor
    for i, n in enumerate([1, 0, 1000, 1 << 20, 3]):
        t = torch.full((n,), float(10 * rank + i))
        got = torch.empty(n)
        if rank == 0:
            dist.send(t, dst=1)
            dist.recv(got, src=1)
        else:
            dist.recv(got, src=0)
            dist.send(t, dst=0)
        assert torch.all(got == float(10 * peer + i)), (rank, i)
    # exchange patterns that an unbuffered rendezvous could wedge on: both post the send first; opposite orders
    a, b = torch.arange(4096.0) + rank, torch.empty(4096)
    ws = [dist.isend(a, peer), dist.irecv(b, peer)]
    ws[1].wait(), ws[0].wait()  # the receive is waited for FIRST: progress must also serve the queued send
    assert torch.equal(b, torch.arange(4096.0) + peer)
    c, d = torch.arange(777.0) * (rank + 2), torch.empty(777)
    ws = [dist.irecv(d, peer), dist.isend(c, peer)] if rank == 0 else [dist.isend(c, peer), dist.irecv(d, peer)]
    for w in ws:
        w.wait()
    assert torch.equal(d, torch.arange(777.0) * (peer + 2))
    for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, a, peer), dist.P2POp(dist.irecv, b, peer)]):
        w.wait()
    # many operations in flight, matched in order
    outs = [torch.empty(64) for _ in range(16)]
    rs = [dist.irecv(o, peer) for o in outs]
    ss = [dist.isend(torch.full((64,), float(100 * rank + k)), peer) for k in range(16)]
    for w in rs + ss:
        w.wait()
    assert all(torch.all(o == float(100 * peer + k)) for k, o in enumerate(outs))
    # a size mismatch is an error on the sender, not silent corruption
    if rank == 0:
        try:
            dist.send(torch.zeros(10), dst=1)
            raise SystemExit("size mismatch should fail")
        except RuntimeError as e:
            assert "expects" in str(e), str(e)
    else:
        w = dist.irecv(torch.empty(11), src=0)
        import time
        time.sleep(1.0)
    print(f"DIRECT_OK {rank}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
