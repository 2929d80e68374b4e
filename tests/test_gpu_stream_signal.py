"""Stream-ordered signals with the real hooks: a transfer submitted with a CUDA stream starts only after the kernels
already queued on that stream, and a stream can wait on the device for a transfer."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_transfer_is_ordered_after_the_stream_and_before_its_waiters():
    body = textwrap.dedent("""
        import ctypes, time, torch
        from dlslime_b200 import _lib, _slime_c as C
        _lib.load()
        assert C.stream_hooks_installed()
        n = 1 << 20
        src = torch.zeros(n, dtype=torch.uint8).pin_memory()
        dst = torch.zeros(n, dtype=torch.uint8).pin_memory()
        dev = torch.full((n,), 7, dtype=torch.uint8, device="cuda")
        a, b = C.TcpEndpoint(), C.TcpEndpoint()
        a.register_memory_region("src", src.data_ptr(), 0, n)
        b.register_memory_region("dst", dst.data_ptr(), 0, n)
        ia, ib = a.endpoint_info(), b.endpoint_info()
        assert a.connect(ib) == 0 and b.connect(ia) == 0
        for name, info in ib["mr_info"].items():
            a.register_remote_memory_region(name, info)
        s = torch.cuda.Stream()
        lh, rh = a.get_mr_handle("src"), a.get_remote_mr_handle("dst")
        # warm-up: first launches load modules and allocate the pinned words
        with torch.cuda.stream(s):
            w = a.write([(lh, rh, 0, 0, 4096)], stream=s.cuda_stream)
            w.wait_on_stream()
        assert w.wait(20) == 0
        torch.cuda.synchronize()
        dst.zero_()
        for trial in range(3):
            fill = 7 + trial
            with torch.cuda.stream(s):
                dev.fill_(fill)
                torch.cuda._sleep(200_000_000)            # ~0.1 s of device time in front of the producer copy
                src.copy_(dev, non_blocking=True)         # the producer: fills the staging buffer on the stream
                gate = torch.cuda.Event()
                gate.record(s)
                f = a.write([(lh, rh, 0, 0, n)], stream=s.cuda_stream)
                f.wait_on_stream()                        # consumers queued on the stream see the transferred bytes
                back = torch.empty(n, dtype=torch.uint8, device="cuda")
                back.copy_(dst, non_blocking=True)
            # the operation cannot be done while the stream has not reached the point where it was submitted
            early = f.done() and not gate.query()
            assert not early, "the transfer completed before its stream reached the submission point"
            assert f.wait(20) == 0
            s.synchronize()
            assert bool((dst == fill).all()), "the transfer read the staging buffer before the producer had filled it"
            assert bool((back == fill).all()), "the consumer on the stream ran before the transfer had completed"
        a.shutdown(); b.shutdown()
        print("ok")
    """)
    env = dict(os.environ, PYTHONPATH=REPO, SLIME_BYPASS_DEVICE_SIGNAL="0")
    r = subprocess.run([sys.executable, "-c", body], env=env, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_stream_wait_that_runs_out_is_reported():
    """A word that nobody sets and a 20 ms limit: the one-thread wait kernel gives up, the stream continues, and the
    signal says so (a future built on it then answers 402 instead of success)."""
    body = textwrap.dedent("""
        import torch
        from dlslime_b200 import _lib, _slime_c as C
        _lib.load()
        s = torch.cuda.Stream()
        sig = C.create_signal(False)
        sig.bind_stream(s.cuda_stream)
        sig.set_stream_wait_limit_ms(20.0)
        assert not sig.stream_wait_timed_out()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s):
            t0.record(s)
            sig.wait_comm_done_on_stream(0b1)      # bit 0 is never set
            t1.record(s)
        s.synchronize()
        ms = t0.elapsed_time(t1)
        assert 15.0 < ms < 500.0, ms
        assert sig.stream_wait_timed_out()
        # a satisfied wait leaves the word alone
        sig.reset_all()
        sig.set_comm_done(0)
        with torch.cuda.stream(s):
            sig.wait_comm_done_on_stream(0b1)
        s.synchronize()
        assert not sig.stream_wait_timed_out()
        print("ok")
    """)
    env = dict(os.environ, PYTHONPATH=REPO, SLIME_BYPASS_DEVICE_SIGNAL="0")
    r = subprocess.run([sys.executable, "-c", body], env=env, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
