"""Low-latency all-to-all over NVLink peer memory (``csrc/kernels/alltoall.cu``).

API shape of the reference's removed op ``AllToAllIntraLLBuffer``
(``dlslime/csrc/python/bind.cpp:515-531`` in the reference: ``buffer_info``, ``connect_full_mesh``,
``get_local_buffer``, ``get_buffer_size_hint``, ``set_max_bs``, ``all_to_all_ll(x, is_transpose, mask, offsets)``).
The reference's tree no longer says what the arguments mean; here they mean:

* ``x`` is ``[world * bs, msg_size]``: rows ``p * bs .. (p + 1) * bs`` go to rank ``p``. The result is
  ``[world * bs, msg_size]`` ordered by source rank (a view of the buffer, valid until the second-next call).
* ``is_transpose=True`` lays the result out as ``[bs, world, msg_size]``: row ``b`` of every source side by side, which is
  the sequence <-> head exchange of Ulysses-style sequence parallelism.
* ``offsets`` (int32 ``[world + 1]`` on the device) replaces the uniform split: rows ``offsets[p] .. offsets[p + 1]`` go
  to rank ``p``, at most ``max_bs`` each. The result is then ``([world, max_bs, msg_size] view, counts [world])``: slot
  ``s`` holds the rows of source ``s`` from its start, and ``counts[s]`` (taken from the flag the source published) says
  how many are valid.
* ``mask`` (int32 ``[world]`` on the device): destinations with ``mask[p] == 0`` get no rows (their count is 0).

``all_to_all_ll_hook`` splits issue and completion like ``all_gather_ll_hook``.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ._common import stream_ptr
from .allgather import AllGatherLLBuffer

_v, _i, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
_cp = ctypes.c_char_p
_lib.declare("slime_a2a_push", [_cp, _v, _ull, _i, _i, _i, _i, _v, _v, _ull, _v, _i, _i, _v, _v])
_lib.declare("slime_a2a_wait", [_cp, _ull, _v, _v])


class AllToAllLLBuffer(AllGatherLLBuffer):
    """Symmetric buffer of ``2 x world x (max_bs x msg_size)`` elements per rank plus flags; see the module text.

    Construction, ``buffer_info`` / ``connect_full_mesh`` / ``get_local_buffer`` and ``emulated_group`` are those of
    :class:`AllGatherLLBuffer` (the memory layout is the same; the flags carry ``step << 32 | rows`` here).
    """

    @staticmethod
    def get_buffer_size_hint(max_bs: int, msg_size: int, dtype: torch.dtype, world_size: int) -> int:
        """Bytes of symmetric memory one rank needs for these limits."""
        slot = (max_bs * msg_size * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        return 2 * world_size * slot + 4096

    def set_max_bs(self, n: int) -> None:
        """Lower (or restore) the per-destination row limit; the allocation made at construction is the ceiling."""
        if n * self.msg_size * self.itemsize > self.slot_bytes:
            raise ValueError(f"max_bs={n} needs more than the {self.slot_bytes}-byte slots this buffer was built with")
        self.max_bs = int(n)
        self._views.clear()

    def _flags_view(self, step: int) -> torch.Tensor:
        off = self.off_flags + (step & 1) * self.world * 8
        return self.heap.view(off, (self.world,), torch.int64, rank=self.rank)

    def _issue_a2a(self, x: torch.Tensor, is_transpose: bool, mask, offsets, do_wait: bool, max_blocks: int = 0):
        if not (x.is_contiguous() and x.dtype == self.dtype and x.dim() == 2 and x.shape[1] == self.msg_size):
            raise ValueError("all_to_all_ll needs a contiguous [rows, msg_size] tensor of the buffer's dtype")
        rows = x.shape[0]
        if offsets is None:
            if rows % self.world:
                raise ValueError(f"{rows} rows do not split evenly over {self.world} ranks; pass offsets")
            bs = rows // self.world
            if bs > self.max_bs:
                raise ValueError(f"{bs} rows per destination exceed max_bs={self.max_bs}")
        else:
            if is_transpose:
                raise ValueError("is_transpose needs the uniform split (no offsets)")
            if not (offsets.is_cuda and offsets.dtype == torch.int32 and offsets.numel() == self.world + 1):
                raise ValueError("offsets must be an int32 CUDA tensor of world + 1 entries")
            bs = 0
        if mask is not None and not (mask.is_cuda and mask.dtype == torch.int32 and mask.numel() == self.world):
            raise ValueError("mask must be an int32 CUDA tensor of world entries")
        self.step += 1
        _lib.call("slime_a2a_push", self._cfg, x.data_ptr(), self.msg_size * self.itemsize, rows, bs, self.max_bs,
                  int(is_transpose), None if offsets is None else offsets.data_ptr(), None if mask is None else mask.data_ptr(),
                  1, self._counter_ptr, int(do_wait), max_blocks, self.status.dev_ptr, torch.cuda.current_stream().cuda_stream)
        return self.step, bs

    def _a2a_result(self, step: int, bs: int, is_transpose: bool, variable: bool):
        half = step & 1
        key = ("a2a", half, bs, is_transpose, variable)
        v = self._views.get(key)
        if v is None:  # building a tensor over raw memory is slow; the handful of shapes in use are kept
            off = self.off_data + half * self.world * self.slot_bytes
            if variable:
                v = (self.heap.view(off, (self.world, self.max_bs, self.msg_size), self.dtype, rank=self.rank), self._flags_view(step))
            else:
                shape = (bs, self.world, self.msg_size) if is_transpose else (self.world * bs, self.msg_size)
                v = self.heap.view(off, shape, self.dtype, rank=self.rank)
            self._views[key] = v
        if variable:
            return v[0], (v[1] & 0xFFFFFFFF).to(torch.int32)
        return v

    def all_to_all_ll(self, x: torch.Tensor, is_transpose: bool = False, mask: torch.Tensor | None = None,
                      offsets: torch.Tensor | None = None):
        """Exchange rows with every rank; returns a view of the buffer (and the counts, with ``offsets``)."""
        step, bs = self._issue_a2a(x, is_transpose, mask, offsets, do_wait=True)
        return self._a2a_result(step, bs, is_transpose, offsets is not None)

    def all_to_all_ll_hook(self, x: torch.Tensor, is_transpose: bool = False, mask: torch.Tensor | None = None,
                           offsets: torch.Tensor | None = None):
        """Issue the stores now; the returned hook waits for the peers and yields the result."""
        step, bs = self._issue_a2a(x, is_transpose, mask, offsets, do_wait=False)

        def hook():
            _lib.call("slime_a2a_wait", self._cfg, 0, self.status.dev_ptr, stream_ptr())
            return self._a2a_result(step, bs, is_transpose, offsets is not None)

        return hook

    # the all-gather entry points of the base class would publish flags in the other format
    def all_gather_ll(self, x):  # pragma: no cover - guard
        raise TypeError("this buffer does all-to-all; use AllGatherLLBuffer for all-gather")

    all_gather_ll_hook = all_gather_ll


# name of the reference's class
AllToAllIntraLLBuffer = AllToAllLLBuffer
