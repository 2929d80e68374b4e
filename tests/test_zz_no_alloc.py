"""The allocation-free batched copy, called through its exported C symbol.

Some embedders of this library cannot let it allocate device memory while serving (their
own pool owns the whole budget, or the host framework forbids allocation on the request
path). For them ``slime_copy_batch_noalloc`` keeps its segment table in a fixed array inside
the library. This test drives that symbol directly with ctypes and checks that it moves
exactly the bytes the regular endpoint transfer moves, on two calls in a row (the second
call reuses the same fixed table with a different batch). Collected last on purpose.
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


def test_noalloc_copy_matches_endpoint_transfer_twice():
    from dlslime_b200 import _lib

    lib = _lib.load()
    fn = lib.slime_copy_batch_noalloc
    fn.restype = ctypes.c_int
    u64p = ctypes.POINTER(ctypes.c_ulonglong)
    fn.argtypes = [u64p, u64p, u64p, ctypes.c_int, ctypes.c_void_p]
    size = 64 << 20
    src = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
    for call, (seed, n_seg) in enumerate([(1, 700), (2, 333)]):
        src_off, dst_off, lens = _batch(seed, n_seg, size)
        expect = torch.zeros(size, dtype=torch.uint8, device="cuda")
        _reference_copy(src, expect, src_off, dst_off, lens)
        got = torch.zeros(size, dtype=torch.uint8, device="cuda")
        d = (dst_off + np.uint64(got.data_ptr())).astype(np.uint64)
        s = (src_off + np.uint64(src.data_ptr())).astype(np.uint64)
        rc = fn(d.ctypes.data_as(u64p), s.ctypes.data_as(u64p), lens.ctypes.data_as(u64p), n_seg,
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, lib.slime_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, expect), f"call {call}: bytes differ from the endpoint transfer"
        assert int(expect.sum().item()) != 0


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
