"""The allocation-free batched copy, called through its exported C symbol.

Some embedders of this library cannot let it allocate device memory while serving (their
own pool owns the whole budget, or the host framework forbids allocation on the request
path). For them ``slime_copy_batch_noalloc`` keeps its segment table in a fixed array inside
the library. This test drives that symbol directly with ctypes and checks that it moves
exactly the bytes the regular endpoint transfer moves, on two calls in a row (the second
call reuses the same fixed table with a different batch), that both agree with a byte-slicing
oracle computed on the CPU (the two kernels share their copy-loop design, so agreement between
them alone would not catch a shared mistake), and that free device memory does not move across
a call. Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _batch(seed, n_seg, size):
    g = np.random.default_rng(seed)
    lens = g.integers(1, 70_000, n_seg)
    lens[::7] = (lens[::7] // 16 + 1) * 16  # some fully aligned segments
    stride = size // n_seg
    src_off = np.arange(n_seg) * stride + g.integers(0, 3, n_seg) * 5
    dst_off = g.permutation(n_seg) * stride + g.integers(0, 2, n_seg) * 16
    lens = np.minimum(lens, stride - 32)
    return src_off.astype(np.uint64), dst_off.astype(np.uint64), lens.astype(np.uint64)


def _reference_copy(src, dst, src_off, dst_off, lens):
    """The same batch through the regular NVLink endpoint (both regions local)."""
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    a, b = NVLinkEndpoint(), NVLinkEndpoint()
    a.register_memory_region(dst.data_ptr(), 0, dst.numel(), "dst")
    b.register_memory_region(src.data_ptr(), 0, src.numel(), "src")
    a.connect(b.endpoint_info())
    fut = a.read([("dst", "src", int(s), int(d), int(n)) for s, d, n in zip(src_off, dst_off, lens)])
    assert fut.wait() == 0
    torch.cuda.synchronize()
    a.close()
    b.close()


u64p = ctypes.POINTER(ctypes.c_ulonglong)


def _entry_point():
    from dlslime_b200 import _lib

    lib = _lib.load()
    fn = lib.slime_copy_batch_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [u64p, u64p, u64p, ctypes.c_int, ctypes.c_void_p]
    return lib, fn


def _call(fn, got, src, src_off, dst_off, lens):
    d = (dst_off + np.uint64(got.data_ptr())).astype(np.uint64)
    s = (src_off + np.uint64(src.data_ptr())).astype(np.uint64)
    lens = np.ascontiguousarray(lens, dtype=np.uint64)
    return fn(d.ctypes.data_as(u64p), s.ctypes.data_as(u64p), lens.ctypes.data_as(u64p), len(lens),
              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _cpu_oracle(src_host, size, src_off, dst_off, lens):
    """What the destination must hold: plain slicing on the CPU, no kernel of this library involved."""
    out = np.zeros(size, dtype=np.uint8)
    for s, d, n in zip(src_off.tolist(), dst_off.tolist(), lens.tolist()):
        out[d:d + n] = src_host[s:s + n]
    return out


def test_noalloc_copy_matches_endpoint_transfer_twice():
    lib, fn = _entry_point()
    size = 64 << 20
    src = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
    src_host = src.cpu().numpy()
    for call, (seed, n_seg) in enumerate([(1, 700), (2, 333)]):
        src_off, dst_off, lens = _batch(seed, n_seg, size)
        expect = torch.zeros(size, dtype=torch.uint8, device="cuda")
        _reference_copy(src, expect, src_off, dst_off, lens)
        got = torch.zeros(size, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(fn, got, src, src_off, dst_off, lens)
        assert rc == 0, lib.slime_last_error()
        torch.cuda.synchronize()
        if call == 1:  # the first call on a device may still load the kernel's module; the second must cost nothing
            assert torch.cuda.mem_get_info()[0] == free_before, "free device memory moved across an allocation-free call"
        assert torch.equal(got, expect), f"call {call}: bytes differ from the endpoint transfer"
        oracle = _cpu_oracle(src_host, size, src_off, dst_off, lens)
        assert np.array_equal(got.cpu().numpy(), oracle), f"call {call}: bytes differ from the CPU oracle"
        assert int(expect.sum().item()) != 0


def test_noalloc_copy_full_table_and_empty_segments():
    """Exactly the maximum number of segments, with zero-length ones at the start, in the middle and at the end."""
    lib, fn = _entry_point()
    lib.slime_copy_batch_noalloc_max_segments.restype = ctypes.c_int
    cap = lib.slime_copy_batch_noalloc_max_segments()
    size = 32 << 20
    stride = size // cap
    g = np.random.default_rng(5)
    lens = g.integers(1, stride - 16, cap).astype(np.uint64)
    for i in (0, 1, cap // 2, cap // 2 + 1, cap - 1):
        lens[i] = 0
    src_off = (np.arange(cap) * stride + g.integers(0, 8, cap)).astype(np.uint64)
    dst_off = (g.permutation(cap) * stride).astype(np.uint64)
    src = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
    got = torch.zeros(size, dtype=torch.uint8, device="cuda")
    assert _call(fn, got, src, src_off, dst_off, lens) == 0, lib.slime_last_error()
    torch.cuda.synchronize()
    oracle = _cpu_oracle(src.cpu().numpy(), size, src_off, dst_off, lens)
    assert np.array_equal(got.cpu().numpy(), oracle)
    # a batch of nothing but empty segments launches nothing and succeeds
    got.zero_()
    zero = np.zeros(8, dtype=np.uint64)
    assert _call(fn, got, src, src_off[:8], dst_off[:8], zero) == 0
    torch.cuda.synchronize()
    assert int(got.sum().item()) == 0


def test_noalloc_copy_rejects_oversized_batch():
    from dlslime_b200 import _lib

    lib = _lib.load()
    lib.slime_copy_batch_noalloc_max_segments.restype = ctypes.c_int
    cap = lib.slime_copy_batch_noalloc_max_segments()
    n = cap + 1
    arr = (ctypes.c_ulonglong * n)()
    fn = lib.slime_copy_batch_noalloc
    fn.restype = ctypes.c_int
    u64p = ctypes.POINTER(ctypes.c_ulonglong)
    fn.argtypes = [u64p, u64p, u64p, ctypes.c_int, ctypes.c_void_p]
    assert fn(arr, arr, arr, n, None) < 0
    lib.slime_last_error.restype = ctypes.c_char_p
    assert b"exceed the fixed table" in lib.slime_last_error()
