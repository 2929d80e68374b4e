"""NVLink endpoint on one GPU: both endpoints live in this process and "remote" regions are local memory.

Covers the three routes of a transfer: one contiguous piece (copy engine, scalar call), a few large pieces
(copy engine from the batched call) and many pieces (one kernel), for read and write, with and without futures.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def pair():
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    size = 48 << 20
    mine = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
    theirs = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
    a, b = NVLinkEndpoint(), NVLinkEndpoint()
    a.register_memory_region(mine.data_ptr(), 0, size, "buf")
    b.register_memory_region(theirs.data_ptr(), 0, size, "buf")
    a.connect(b.endpoint_info())
    yield a, mine, theirs
    torch.cuda.synchronize()
    a.close()
    b.close()


def _apply(expect_dst, src, segs, is_write):
    for roff, loff, n in segs:
        if is_write:  # local -> remote
            expect_dst[roff:roff + n] = src[loff:loff + n]
        else:  # remote -> local
            expect_dst[loff:loff + n] = src[roff:roff + n]


@pytest.mark.parametrize("is_write", [False, True])
@pytest.mark.parametrize("segs", [
    [(5, 3, 1)],  # one unaligned byte
    [(4096, 1 << 20, 100_000)],  # one contiguous piece
    [(0, 24 << 20, 8 << 20), (16 << 20, 8 << 20, 5 << 20), (40 << 20, 0, (4 << 20) + 16)],  # few large pieces
    [(1000 * i + (i % 3), (20 << 20) + 5000 * i + (i % 5), 777 + 16 * i) for i in range(250)],  # many small pieces
    [(0, 0, 0)],  # nothing to move
], ids=["byte", "single", "few-large", "many-small", "empty"])
def test_transfer_routes(pair, segs, is_write):
    ep, mine, theirs = pair
    lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
    if is_write:  # the lists give (source offset, destination offset, length) with disjoint destinations
        segs = [(loff, roff, n) for roff, loff, n in segs]
    dst, src = (theirs, mine) if is_write else (mine, theirs)
    expect = dst.clone()
    _apply(expect, src, segs, is_write)
    op = ep.write if is_write else ep.read
    fut = op([(lh, rh, roff, loff, n) for roff, loff, n in segs])
    assert fut.wait(10.0) == 0, "the completion word never arrived"
    assert torch.equal(dst, expect)
    # the same batch by name and without a future: the caller synchronises the stream, as with the reference's endpoint
    dst.copy_(expect.flip(0))
    expect2 = dst.clone()
    _apply(expect2, src, segs, is_write)
    fut2 = op([("buf", "buf", roff, loff, n) for roff, loff, n in segs], want_future=False)
    torch.cuda.synchronize()
    assert fut2.done() and fut2.wait() == 0
    assert torch.equal(dst, expect2)


def test_out_of_range_piece_is_refused(pair):
    from dlslime_b200._lib import SlimeCudaError

    ep, mine, _ = pair
    lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
    before = mine.clone()
    with pytest.raises(SlimeCudaError):
        ep.read([(lh, rh, (48 << 20) - 8, 0, 16)])  # runs past the remote region
    with pytest.raises(SlimeCudaError):
        ep.read([(lh, 99, 0, 0, 16)])  # unknown remote handle
    with pytest.raises(SlimeCudaError):
        ep.write([(lh, rh, 0, 0, 8 << 20), (lh, rh, 0, (48 << 20) - 1, 8 << 20)])  # second large piece out of range
    torch.cuda.synchronize()
    assert torch.equal(mine, before)


def test_wrapped_and_negative_offsets_are_refused(pair):
    """An offset near 2^64 (what a negative number becomes in an unsigned argument) must not pass the range check
    by wrapping `offset + length`; the refusal happens on the host, before anything is launched."""
    import ctypes

    import numpy as np

    from dlslime_b200 import _lib
    from dlslime_b200._lib import SlimeCudaError

    ep, mine, theirs = pair
    lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
    before_m, before_t = mine.clone(), theirs.clone()
    for bad in [(lh, rh, -16, 0, 32), (lh, rh, 0, -16, 32), (lh, rh, 0, 0, -1)]:
        with pytest.raises(ValueError):
            ep.read([bad])  # scalar route
        with pytest.raises(ValueError):
            ep.write([bad, (lh, rh, 0, 0, 16)])  # table route
    huge = (1 << 64) - 16
    # straight through the C entry points, as a caller without the Python checks would
    lib = _lib.load()
    assert lib.slime_nvlink_ep_copy1(ep._h, lh, rh, ctypes.c_ulonglong(huge), 0, 32, 0, None, 0, None) < 0
    assert lib.slime_nvlink_ep_copy1(ep._h, lh, rh, 0, ctypes.c_ulonglong(huge), 32, 1, None, 0, None) < 0
    for row in [(lh, rh, huge, 0, 32), (lh, rh, 0, huge, 32), (lh, rh, 16, 16, huge)]:
        arr = np.asarray([row, (lh, rh, 0, 0, 16)] * 8, dtype=np.uint64)  # 16 pieces: the kernel route
        with pytest.raises(SlimeCudaError):
            ep.read(arr)
    torch.cuda.synchronize()
    assert torch.equal(mine, before_m) and torch.equal(theirs, before_t)


def test_write_with_imm_after_single_piece(pair):
    """The immediate travels behind a copy-engine write in stream order (self-connected pair shares one mailbox owner)."""
    ep, mine, theirs = pair
    lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
    expect = theirs.clone()
    expect[64:64 + 4096] = mine[128:128 + 4096]
    fut = ep.write_with_imm([(lh, rh, 64, 128, 4096)], imm_data=0xC0DE)
    assert fut.wait(10.0) == 0
    assert torch.equal(theirs, expect)


def test_transfers_are_accounted_as_an_nvlink_link():
    """With the counters on, an endpoint is one link of kind "nvlink": one submit per user operation, completed bytes
    when the future first sees its word."""
    from dlslime_b200 import _slime_c
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    _slime_c.obs_set_enabled_for_test(True)
    _slime_c.obs_reset_for_test()
    try:
        size = 1 << 20
        mine = torch.zeros(size, dtype=torch.uint8, device="cuda")
        theirs = torch.randint(0, 255, (size,), dtype=torch.uint8, device="cuda")
        a, b = NVLinkEndpoint(), NVLinkEndpoint()
        a.register_memory_region(mine.data_ptr(), 0, size, "buf")
        b.register_memory_region(theirs.data_ptr(), 0, size, "buf")
        a.connect(b.endpoint_info())
        lh, rh = a.get_mr_handle("buf"), a.get_remote_mr_handle("buf")
        fut = a.read([(lh, rh, 4096 * i, 4096 * i, 1000 + i) for i in range(3)])
        assert fut.wait(10.0) == 0
        assert a.write([(lh, rh, 0, 0, 512)]).wait(10.0) == 0
        assert a.write_with_imm([(lh, rh, 8192, 8192, 64)], imm_data=7).wait(10.0) == 0
        a.read([(lh, rh, 0, 0, 256)], want_future=False)
        torch.cuda.synchronize()
        snap = _slime_c.obs_snapshot()
        link = next(n for n in snap["nics"] if n["nic"] == f"nvlink:gpu{torch.cuda.current_device()}")
        assert link["kind"] == "nvlink"
        rd, wr, wi = link["by_op"]["read"], link["by_op"]["write"], link["by_op"]["write_with_imm"]
        assert (rd["batch"], rd["assign"], rd["submitted_bytes"], rd["completed_bytes"]) == (2, 4, 3003 + 256, 3003 + 256)
        assert (wr["batch"], wr["assign"], wr["completed_bytes"]) == (1, 1, 512)
        assert (wi["batch"], wi["assign"], wi["completed_bytes"]) == (1, 1, 64)
        assert link["pending_ops"] == 0 and snap["summary"]["pending_ops"] == 0
        a.close()
        b.close()
    finally:
        _slime_c.obs_reset_for_test()
        _slime_c.obs_set_enabled_for_test(False)
