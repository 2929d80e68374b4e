"""The C function table over the endpoints (csrc/include/slime_bridge.h), driven through ctypes the way native code would."""
import ctypes as C

from dlslime_b200 import _slime_c


class Bridge(C.Structure):
    _fields_ = [
        ("version", C.c_int),
        ("endpoint_create", C.CFUNCTYPE(C.c_void_p, C.c_char_p, C.c_char_p, C.c_int, C.c_char_p, C.c_size_t)),
        ("endpoint_destroy", C.CFUNCTYPE(None, C.c_void_p)),
        ("endpoint_info", C.CFUNCTYPE(C.c_void_p, C.c_void_p)),
        ("endpoint_connect", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_char_p, C.c_char_p, C.c_size_t)),
        ("endpoint_kind", C.CFUNCTYPE(C.c_char_p, C.c_void_p)),
        ("send", C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t)),
        ("recv", C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t)),
        ("future_wait", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int64)),
        ("future_done", C.CFUNCTYPE(C.c_int, C.c_void_p)),
        ("future_free", C.CFUNCTYPE(None, C.c_void_p)),
        ("free_string", C.CFUNCTYPE(None, C.c_void_p)),
    ]


def _info(b, ep):
    p = b.endpoint_info(ep)
    text = C.string_at(p)
    b.free_string(p)
    return text


def test_send_recv_and_timeout_through_the_table():
    b = Bridge.from_address(_slime_c.bridge_table())
    assert b.version == 1
    err = C.create_string_buffer(256)
    x = b.endpoint_create(b"tcp", b"127.0.0.1", 0, err, 256)
    y = b.endpoint_create(b"tcp", b"127.0.0.1", 1, err, 256)
    assert x and y, err.value
    assert b.endpoint_kind(x) == b"tcp"
    ix, iy = _info(b, x), _info(b, y)
    assert b.endpoint_connect(x, iy, err, 256) == 0 and b.endpoint_connect(y, ix, err, 256) == 0, err.value
    src = C.create_string_buffer(bytes(range(200)) * 50, 10_000)
    dst = C.create_string_buffer(10_000)
    r = b.recv(y, C.addressof(dst), 10_000)
    s = b.send(x, C.addressof(src), 10_000)
    assert b.future_wait(s, 10_000) == 0 and b.future_wait(r, 10_000) == 0
    assert b.future_done(r) == 1 and dst.raw == src.raw
    b.future_free(s)
    b.future_free(r)
    # a receive nobody answers runs into its limit (402) and the endpoint stays usable for shutdown
    lonely = b.recv(y, C.addressof(dst), 16)
    assert b.future_done(lonely) == 0
    assert b.future_wait(lonely, 100) == 402
    b.endpoint_destroy(x)
    assert b.future_wait(lonely, 5_000) in (402, 403)  # failed by the peer's exit or by our own shutdown below
    b.endpoint_destroy(y)
    b.future_free(lonely)


def test_bad_requests_report_instead_of_crashing():
    b = Bridge.from_address(_slime_c.bridge_table())
    err = C.create_string_buffer(256)
    ep = b.endpoint_create(b"tcp", b"", 0, err, 256)
    assert ep
    assert b.endpoint_connect(ep, b"{not json", err, 256) != 0 and err.value
    b.endpoint_destroy(ep)


def test_rdma_endpoints_through_the_table_on_the_software_fabric():
    """transport "rdma" builds RC endpoints (here on the in-process fabric); mixing kinds is refused with a message."""
    import os
    import subprocess
    import sys
    import textwrap

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = textwrap.dedent("""
        import ctypes as C, sys
        sys.path.insert(0, %r)
        from test_bridge import Bridge, _info
        from dlslime_b200 import _slime_c
        b = Bridge.from_address(_slime_c.bridge_table())
        err = C.create_string_buffer(256)
        x, y = b.endpoint_create(b"rdma", b"", 0, err, 256), b.endpoint_create(b"rdma", b"", 1, err, 256)
        t = b.endpoint_create(b"tcp", b"127.0.0.1", 2, err, 256)
        assert x and y and t and b.endpoint_kind(x) == b"rdma" and b.endpoint_kind(t) == b"tcp"
        ix, iy, it = _info(b, x), _info(b, y), _info(b, t)
        assert b.endpoint_connect(x, it, err, 256) != 0 and err.value   # an RC endpoint cannot take a TCP description
        assert b.endpoint_connect(x, iy, err, 256) == 0 and b.endpoint_connect(y, ix, err, 256) == 0
        src = C.create_string_buffer(bytes(range(250)) * 400, 100_000)
        dst = C.create_string_buffer(100_000)
        r, s = b.recv(y, C.addressof(dst), 100_000), b.send(x, C.addressof(src), 100_000)
        assert b.future_wait(s, 10_000) == 0 and b.future_wait(r, 10_000) == 0 and dst.raw == src.raw
        for f in (s, r):
            b.future_free(f)
        for e in (x, y, t):
            b.endpoint_destroy(e)
        print("ok")
    """ % os.path.join(repo, "tests"))
    res = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, PYTHONPATH=repo, SLIME_RDMA_PROVIDER="loopback"),
                         capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout[-1500:] + res.stderr[-1500:]
