"""Symmetric device memory: one region per rank, mapped into every rank.

Each rank allocates a ``cudaMalloc`` region (outside the torch caching
allocator), exports its 64-byte CUDA IPC handle, and maps every peer's region, so
kernels can address any rank's buffer with plain loads and stores over NVLink.
Handles travel through a ``torch.distributed`` process group (any backend), the
same bootstrap the reference's NVLink example uses
(``examples/python/p2p_nvlink.py:20-61`` in the reference); a PeerAgent or any other
out-of-band channel can carry them as well, see ``export_info`` / ``connect``.

``SymmetricHeap.emulated(n)`` creates ``n`` regions on ONE device. That mode backs
the single-GPU tests of multi-rank protocols: kernels are replayed rank by rank
and every wait finds its flag already published.

Guard bands (debugging aid, ``SLIME_HEAP_GUARD=1`` in the environment of EVERY rank, since
offsets must stay identical across ranks): each reservation is followed by a 256-byte band
filled with ``0xA5`` (one more band sits in front of the first reservation);
``check_guards()`` lists the bands of this rank's region(s) that no longer hold the pattern, i.e.
where a kernel of this or of another rank wrote outside its buffer.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

from .. import _lib


class _RawCudaBuffer:
    """Adapter that lets torch view raw device memory without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device | int | None = None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes), device=dev)


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


GUARD_BYTES = 256
GUARD_BYTE = 0xA5
_GUARD_SLACK = 64 << 10  # room for 256 bands on top of what the caller asked for


class SymmetricHeap:
    """A region of ``nbytes`` on every rank plus the peer mappings."""

    def __init__(self, nbytes: int, group=None, _emulated_world: int = 0):
        import torch.distributed as dist

        self.guard = os.environ.get("SLIME_HEAP_GUARD", "0") not in ("", "0")
        self.nbytes = _align(int(nbytes) + (_GUARD_SLACK if self.guard else 0), 1 << 21)
        self._guards: list[int] = []
        self._owned: list[int] = []
        self._opened: list[int] = []
        self._cursor = 0
        self.group = group
        if _emulated_world:
            self.world, self.rank = _emulated_world, 0
            self.peer_ptrs = [self._alloc()[0] for _ in range(_emulated_world)]
            self.local_ptr = self.peer_ptrs[0]
            self.emulated = True
            return
        self.emulated = False
        if dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        else:
            self.world, self.rank = 1, 0
        self.local_ptr, handle = self._alloc()
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        if self.world > 1:
            infos = [None] * self.world
            dist.all_gather_object(infos, {"rank": self.rank, "ipc_handle": list(handle), "length": self.nbytes}, group=group)
            self.connect(infos)
            dist.barrier(group=group)

    # -- construction helpers -------------------------------------------------
    @classmethod
    def emulated(cls, world: int, nbytes: int) -> "SymmetricHeap":
        return cls(nbytes, _emulated_world=world)

    def _alloc(self):
        p = ctypes.c_void_p()
        h = (ctypes.c_ubyte * 64)()
        _lib.call("slime_symm_alloc", self.nbytes, ctypes.byref(p), h)
        self._owned.append(p.value)
        return p.value, bytes(h)

    def export_info(self) -> dict:
        h = (ctypes.c_ubyte * 64)()
        _lib.call("slime_ipc_get_handle", ctypes.c_void_p(self.local_ptr), h, None, None)
        return {"rank": self.rank, "ipc_handle": list(bytes(h)), "length": self.nbytes}

    def connect(self, infos: Sequence[dict]) -> None:
        """Map every peer's region. ``infos[r]`` is rank r's ``export_info()``."""
        for info in infos:
            r = info["rank"]
            if r == self.rank:
                continue
            if info["length"] != self.nbytes:
                raise ValueError(f"rank {r} exported {info['length']} bytes, expected {self.nbytes}")
            h = (ctypes.c_ubyte * 64)(*[b & 0xFF for b in info["ipc_handle"]])
            p = ctypes.c_void_p()
            _lib.call("slime_ipc_open", h, ctypes.byref(p))
            self._opened.append(p.value)
            self.peer_ptrs[r] = p.value

    # -- carving --------------------------------------------------------------
    def reserve(self, nbytes: int, align: int = 256) -> int:
        """Reserve ``nbytes`` at the same offset on every rank; returns the offset."""
        if self.guard and not self._guards:
            self._place_guard(0)
            self._cursor = GUARD_BYTES
        off = _align(self._cursor, align)
        end = off + nbytes
        if self.guard:
            end = _align(end, 16) + GUARD_BYTES
        if end > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {end}, have {self.nbytes}")
        if self.guard:
            self._place_guard(end - GUARD_BYTES)
        self._cursor = end
        return off

    def _place_guard(self, off: int) -> None:
        self._guards.append(off)
        for p in self._owned:
            tensor_from_ptr(p + off, GUARD_BYTES).fill_(GUARD_BYTE)

    def check_guards(self) -> list[tuple[int, int]]:
        """``(region index, band offset)`` of every damaged guard band in the regions this process owns
        (one region, or all of them for an emulated group). Synchronises the device."""
        torch.cuda.synchronize()
        bad = []
        for i, p in enumerate(self._owned):
            for off in self._guards:
                if not bool((tensor_from_ptr(p + off, GUARD_BYTES) == GUARD_BYTE).all()):
                    bad.append((i, off))
        return bad

    def view(self, offset: int, shape, dtype: torch.dtype, rank: int | None = None) -> torch.Tensor:
        """Tensor view of ``[offset, offset + prod(shape) * itemsize)`` in rank ``rank``'s region."""
        r = self.rank if rank is None else rank
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if offset + nbytes > self.nbytes:
            raise ValueError("view exceeds the symmetric region")
        raw = tensor_from_ptr(self.peer_ptrs[r] + offset, max(nbytes, 1))
        return raw[:nbytes].view(dtype).reshape(tuple(shape))

    def zero_(self) -> None:
        for p in self._owned:
            _lib.call("slime_memset_async", ctypes.c_void_p(p), 0, self.nbytes, None)
        torch.cuda.synchronize()
        for p in self._owned:
            for off in self._guards:
                tensor_from_ptr(p + off, GUARD_BYTES).fill_(GUARD_BYTE)

    def close(self) -> None:
        torch.cuda.synchronize()
        for p in self._opened:
            _lib.call("slime_ipc_close", ctypes.c_void_p(p))
        self._opened.clear()
        for p in self._owned:
            _lib.call("slime_symm_free", ctypes.c_void_p(p))
        self._owned.clear()

    def __del__(self):
        try:
            if self._owned or self._opened:
                self.close()
        except Exception:
            pass
