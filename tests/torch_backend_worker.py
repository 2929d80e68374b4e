"""Worker of test_torch_backend.py: two CPU ranks exchange tensors through the "dlslime" c10d backend."""
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
    for i in range(4):  # ordered pairs
        t = torch.full((1000 + i,), float(10 * rank + i))
        if rank == 0:
            dist.send(t, dst=1)
            got = torch.empty(1000 + i)
            dist.recv(got, src=1)
        else:
            got = torch.empty(1000 + i)
            dist.recv(got, src=0)
            dist.send(t, dst=0)
        assert torch.all(got == float(10 * peer + i)), (rank, i, got[:3])
    a, b = torch.arange(64.0) + rank, torch.empty(64)
    ops = [dist.P2POp(dist.isend, a, peer), dist.P2POp(dist.irecv, b, peer)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    assert torch.equal(b, torch.arange(64.0) + peer)
    try:
        dist.all_reduce(torch.ones(1))
        raise SystemExit("all_reduce should not be supported")
    except (NotImplementedError, RuntimeError) as e:
        assert "not support" in str(e), str(e)  # "is not supported" (Python form) / "does not support allreduce" (c10d::Backend)
    several = [torch.full((17,), float(rank)), torch.full((5, 3), float(rank) + 0.5)]  # every tensor of a list is moved
    got = [torch.empty(17), torch.empty(5, 3)]
    pg = dist.distributed_c10d._get_default_group()
    if rank == 0:
        pg.send(several, 1, 0).wait()
        pg.recv(got, 1, 0).wait()
    else:
        pg.recv(got, 0, 0).wait()
        pg.send(several, 0, 0).wait()
    assert torch.all(got[0] == float(peer)) and torch.all(got[1] == float(peer) + 0.5)
    if "--cuda" in sys.argv:  # device tensors go device to device (CUDA IPC); both ranks may share one GPU
        dev = torch.device("cuda", 0)
        x = torch.arange(4096, dtype=torch.float32, device=dev) * (rank + 1)
        y = torch.empty(4096, dtype=torch.float32, device=dev)
        if rank == 0:
            dist.send(x, dst=1)
            dist.recv(y, src=1)
        else:
            dist.recv(y, src=0)
            dist.send(x, dst=0)
        torch.cuda.synchronize()
        assert torch.equal(y, torch.arange(4096, dtype=torch.float32, device=dev) * (peer + 1))
        # a larger tensor produced by a kernel right before the send, and an exchange with both sends posted first
        big = torch.randn(1 << 22, device=dev)
        big.mul_(rank + 1.5)
        back = torch.empty_like(big)
        ws = [dist.isend(big, peer), dist.irecv(back, peer)]
        ws[1].wait(), ws[0].wait()
        torch.cuda.synchronize()
        ref = [None, None]
        ref[rank] = big
        chk = torch.empty(2, device=dev)
        chk[0], chk[1] = big.double().sum().float(), back.double().sum().float()
        sums = chk.cpu().tolist()
        other = torch.empty(2)
        mine = torch.tensor(sums)
        if rank == 0:
            dist.send(mine, dst=1); dist.recv(other, src=1)
        else:
            dist.recv(other, src=0); dist.send(mine, dst=0)
        assert abs(other[0].item() - sums[1]) <= 1e-3 * max(1.0, abs(sums[1])), "the received tensor is not what the peer sent"
        if os.environ.get("SLIME_BACKEND_DIRECT", "auto") == "auto":
            c = pg.counters
            assert c["direct_sends"] >= 2 and c["direct_recvs"] >= 2 and c["staged_fallbacks"] == 0, c
    # wait(timeout) is honoured: a receive that nobody sends ends with status 402 instead of blocking
    import time
    from datetime import timedelta

    if rank == 0:
        w = pg.recv([torch.empty(8)], 1, 0)
        t0 = time.monotonic()
        try:
            w.wait(timedelta(milliseconds=300))
            raise SystemExit("the unmatched recv should have timed out")
        except RuntimeError as e:
            assert "402" in str(e) and time.monotonic() - t0 < 5.0, str(e)
    else:
        time.sleep(1.5)  # stay connected while rank 0 waits
    print(f"BACKEND_OK {rank} {dlslime_b200.torch_backend.implementation()}", flush=True)
    os._exit(0)  # skip the default teardown barrier, which this backend does not implement


if __name__ == "__main__":
    main()
