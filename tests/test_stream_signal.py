"""Stream-ordered signals with a fake CUDA layer: the four hooks are ctypes callbacks and a "stream" is a list of
deferred actions, so the ordering contract is checked without a GPU. (A GPU test runs the real hooks.)"""
import os
import subprocess
import sys
import textwrap

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_transfer_waits_for_the_stream_and_stream_can_wait_for_the_transfer():
    body = textwrap.dedent("""
        import ctypes
        from ctypes import CFUNCTYPE, POINTER, c_int, c_ulonglong, c_void_p
        from dlslime_b200 import _slime_c as C

        keep, stream_queue, waits = [], [], []

        @CFUNCTYPE(c_int, c_ulonglong, POINTER(c_void_p), POINTER(c_void_p))
        def alloc(n, host, dev):
            b = (ctypes.c_ulonglong * n)()
            keep.append(b)
            host[0] = ctypes.addressof(b); dev[0] = ctypes.addressof(b)    # "device" address == host address here
            return 0

        @CFUNCTYPE(c_int, c_void_p)
        def free(p):
            return 0

        @CFUNCTYPE(c_int, c_void_p, c_void_p, c_ulonglong)
        def record(stream, word, value):
            stream_queue.append(("record", stream, word, value))
            return 0

        @CFUNCTYPE(c_int, c_void_p, c_void_p, c_ulonglong, c_ulonglong, c_void_p)
        def wait(stream, word, mask, limit, timeout_word):
            stream_queue.append(("wait", stream, word, mask))
            waits.append((limit, timeout_word))
            return 0

        addr = lambda f: ctypes.cast(f, c_void_p).value
        assert not C.stream_hooks_installed()
        C.install_stream_hooks(addr(alloc), addr(free), addr(record), addr(wait))
        assert C.stream_hooks_installed()

        # the signal on its own
        s = C.create_signal(False)
        s.bind_stream(77)
        s.record_gpu_ready()
        assert not s.is_gpu_ready() and stream_queue[-1][0] == "record" and stream_queue[-1][1] == 77
        kind, _, word, value = stream_queue.pop()
        ctypes.c_ulonglong.from_address(word).value = value               # the stream "executes" the write
        assert s.is_gpu_ready()
        s.set_comm_done(0); s.set_comm_done(3)
        assert s.get_comm_done_mask() == 0b1001
        s.wait_comm_done_on_stream(0b1001)
        kind, _, word, mask = stream_queue.pop()
        assert kind == "wait" and ctypes.c_ulonglong.from_address(word).value & mask == mask

        # through an endpoint: nothing moves until the stream has run
        a, b = C.TcpEndpoint(), C.TcpEndpoint()
        n = 4096
        src = ctypes.create_string_buffer(b"x" * n, n); dst = ctypes.create_string_buffer(n)
        a.register_memory_region("src", ctypes.addressof(src), 0, n)
        b.register_memory_region("dst", ctypes.addressof(dst), 0, n)
        ia, ib = a.endpoint_info(), b.endpoint_info()
        assert a.connect(ib) == 0 and b.connect(ia) == 0
        for name, info in ib["mr_info"].items():
            a.register_remote_memory_region(name, info)
        f = a.write([(a.get_mr_handle("src"), a.get_remote_mr_handle("dst"), 0, 0, n)], stream=5)
        assert f.wait(0.3) == 402 and dst.raw == bytes(n), "the transfer ran before its stream reached the ready mark"
        kind, stream, word, value = stream_queue.pop()
        assert (kind, stream) == ("record", 5)
        ctypes.c_ulonglong.from_address(word).value = value
        assert f.wait(10) == 0 and dst.raw == src.raw
        f.wait_on_stream()
        kind, stream, word, mask = stream_queue.pop()
        assert (kind, stream) == ("wait", 5) and ctypes.c_ulonglong.from_address(word).value & mask == mask
        assert waits[-1][0] == 1_000_000_000 and not f.stream_wait_timed_out()

        # a stream-ordered wait that runs into its limit: the "device" sets the timeout word, and the future must say
        # 402 although the transfer itself succeeded (the stream's consumers ran without the data)
        f2 = a.write([(a.get_mr_handle("src"), a.get_remote_mr_handle("dst"), 0, 0, n)], stream=5)
        kind, stream, word, value = stream_queue.pop()
        ctypes.c_ulonglong.from_address(word).value = value
        assert f2.wait(10) == 0
        f2.wait_on_stream(limit_ms=20)
        limit, timeout_word = waits[-1]
        assert limit == 20_000_000
        ctypes.c_ulonglong.from_address(timeout_word).value = 1          # what the bounded kernel does when it gives up
        assert f2.stream_wait_timed_out() and f2.wait(10) == 402
        a.shutdown(); b.shutdown()
        print("ok")
    """)
    env = dict(os.environ, PYTHONPATH=REPO, SLIME_BYPASS_DEVICE_SIGNAL="0")
    r = subprocess.run([sys.executable, "-c", body], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
