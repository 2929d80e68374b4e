"""Assignment model, splitters, signals and memory pools of the host runtime (no GPU, no network)."""
import ctypes
import threading
import time

import pytest

from dlslime_b200 import _slime_c as c


def test_assignment_fields_and_tuple_order():
    a = c.Assignment(11, 22, 4096, 8192, 2048)
    assert (a.mr_key, a.remote_mr_key, a.target_offset, a.source_offset, a.length) == (11, 22, 4096, 8192, 2048)
    assert a.to_tuple() == (11, 22, 4096, 8192, 2048)
    b = c.Assignment(7, 1, 2, 3)  # one key for both sides
    assert (b.mr_key, b.remote_mr_key) == (7, 7)
    assert '"target_offset":4096' in a.dump()


def test_split_by_max_length_keeps_offsets_in_step():
    out = c.split_assign_by_max_length([c.Assignment(1, 2, 10, 20, 2500), c.Assignment(1, 2, 0, 0, 5)], 1000)
    assert [(x.target_offset, x.source_offset, x.length) for x in out] == [(10, 20, 1000), (1010, 1020, 1000), (2010, 2020, 500), (0, 0, 5)]


def test_split_by_step_and_nsplit():
    batch = [c.Assignment(1, 1, i, i, 1) for i in range(10)]
    groups = c.split_assign_by_step(batch, 4)
    assert [len(g) for g in groups] == [4, 4, 2]
    assert [len(g) for g in c.nsplit_assign_by_step(batch, 3)] == [4, 4, 2]
    assert c.split_assign_by_step([], 4) == [] and c.nsplit_assign_by_step(batch, 0) == []


def test_opcode_names_match_public_api():
    assert {n for n in dir(c.OpCode) if n.isupper()} >= {"READ", "WRITE", "WRITE_WITH_IMM_DATA", "SEND", "RECV"}


def test_signal_mask_wait_timeout_and_force():
    s = c.create_signal()
    assert s.wait(0b11, 0.05) is False  # nothing set: times out instead of hanging
    s.set_comm_done(0)
    assert s.wait(0b11, 0.05) is False
    threading.Timer(0.05, lambda: s.set_comm_done(1)).start()
    t0 = time.monotonic()
    assert s.wait(0b11, 2.0) is True and time.monotonic() - t0 < 1.0
    s.reset_all()
    assert s.get_comm_done_mask() == 0
    s.force_complete()
    assert s.wait(0b1111, 0.5) is True  # forced completion wakes any waiter


def test_memory_pool_idempotent_grow_and_unregister():
    pool = c.MemoryPool()
    buf = ctypes.create_string_buffer(8192)
    p = ctypes.addressof(buf)
    h = pool.register_memory_region(p, 4096, "kv")
    assert pool.register_memory_region(p, 4096, "kv") == h  # same pointer, same handle
    assert pool.register_memory_region(p, 8192, "kv") == h  # grown region keeps its handle
    assert pool.mr_info()["kv"]["length"] == 8192 and pool.mr_info()["kv"]["handle"] == h
    h2 = pool.register_memory_region(p + 64, 128)  # auto name
    assert h2 != h and any(k.startswith("auto_0x") for k in pool.mr_info())
    assert pool.unregister_memory_region("kv") == 0
    assert pool.get_handle("kv") == -1 and pool.unregister_memory_region("kv") == -1
    assert pool.unregister_memory_region(h2) == 0 and pool.live_count() == 0
    h3 = pool.register_memory_region(p, 16, "kv")
    assert h3 not in (h, h2), "handles are never reused"


def test_ascend_endpoint_is_an_interface_stub():
    ep = c.AscendDirectEndpoint()
    ep.init("127.0.0.1", 16000)
    assert ep.register_memory_region(0x1000, 0, 64, "buf") == 0
    info = ep.endpoint_info()
    assert info["host"] == "127.0.0.1" and info["mr_info"]["buf"]["length"] == 64
    with pytest.raises(RuntimeError, match="not available"):
        ep.connect(info)


def test_nvtx_ranges_are_compiled_in_where_the_toolkit_headers_exist():
    """The host runtime wraps its signal operations in NVTX ranges when it was built with the CUDA toolkit's headers on
    the include path (they are header-only); without them the macros are no-ops and the flag says so."""
    import pathlib

    from dlslime_b200 import _build, _slime_c

    assert isinstance(_slime_c._BUILD_NVTX, bool)
    if _build._cuda_include():
        assert _slime_c._BUILD_NVTX
    text = (pathlib.Path(_build.CSRC) / "host" / "engine" / "signal.h").read_text()
    assert text.count("SLIME_NVTX_RANGE(") >= 3
