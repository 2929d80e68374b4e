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

Multicast-capable heaps (``multicast=True`` / ``None``): the region comes from the virtual-memory-management API
instead (``csrc/kernels/symm_vmm.cu``): every rank creates its region with ``cuMemCreate``, the regions travel as POSIX
file descriptors over Unix sockets (``SCM_RIGHTS``), every rank maps every peer, and all regions are bound to one NVLink
multicast object whose mapping is ``mc_ptr``. A ``multimem.st`` to ``mc_ptr + offset`` lands at ``offset`` in every
rank's region; the peer pointers work as before. ``multicast=None`` tries this and falls back to the IPC heap when the
GPUs (or the group: all ranks must share a node and an NVSwitch) cannot do it; every rank takes the same decision.
``close()`` unmaps and unbinds before anything is released, and runs at interpreter exit for heaps that are still
open: a rank must never leave while its memory is bound to a multicast object that others use.

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

    def __init__(self, nbytes: int, group=None, _emulated_world: int = 0, multicast: bool | None = False):
        import torch.distributed as dist

        self.guard = os.environ.get("SLIME_HEAP_GUARD", "0") not in ("", "0")
        self.nbytes = _align(int(nbytes) + (_GUARD_SLACK if self.guard else 0), 1 << 21)
        self._guards: list[int] = []
        self._owned: list[int] = []
        self._opened: list[int] = []
        self._cursor = 0
        self.group = group
        self.mc_ptr = 0  # address of the multicast mapping (0: plain peer pointers only)
        self._vmm = None  # state of a VMM / multicast heap, see _init_vmm
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
        if os.environ.get("SLIME_SYMM_MULTICAST", "") == "0":
            multicast = False
        if multicast is not False and self.world > 1 and self._init_vmm(required=multicast is True):
            return
        self.local_ptr, handle = self._alloc()
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        if self.world > 1:
            infos = [None] * self.world
            dist.all_gather_object(infos, {"rank": self.rank, "ipc_handle": list(handle), "length": self.nbytes}, group=group)
            self.connect(infos)
            dist.barrier(group=group)

    # -- VMM + multicast ------------------------------------------------------
    def _all_agree(self, ok: bool) -> bool:
        import torch.distributed as dist

        votes = [None] * self.world
        dist.all_gather_object(votes, bool(ok), group=self.group)
        return all(votes)

    def _exchange_fds(self, tag: str, fds: list[int]) -> dict[int, list[int]]:
        """Send ``fds`` to every other rank of the group and receive theirs: one abstract Unix socket per rank,
        descriptors as ancillary data. Returns ``{rank: [fd, ...]}`` (duplicates owned by this process)."""
        import socket
        import struct as _struct

        import torch.distributed as dist

        name = lambda r: f"\0slime-vmm-{tag}-{r}"  # noqa: E731  (abstract namespace: nothing to unlink)
        # No exception may leave this function between the two barriers: a rank that raised would leave the others
        # waiting in a collective. Errors are kept and raised at the end, after every rank has passed both.
        error: Exception | None = None
        srv = None
        try:
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            srv.bind(name(self.rank))
            srv.listen(self.world)
            srv.settimeout(30.0)
        except Exception as e:  # noqa: BLE001
            error = e
        dist.barrier(group=self.group)  # everybody listens before anybody connects
        got: dict[int, list[int]] = {}
        try:
            for r in range(self.world):
                if r == self.rank:
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                    c.settimeout(30.0)
                    c.connect(name(r))
                    socket.send_fds(c, [_struct.pack("<ii", self.rank, len(fds))], fds)
            for _ in range(self.world - 1):
                if srv is None:
                    break
                conn, _addr = srv.accept()
                with conn:
                    conn.settimeout(30.0)
                    msg, rfds, _flags, _a = socket.recv_fds(conn, 8, 8)
                    src, n = _struct.unpack("<ii", msg)
                    got[src] = list(rfds)
                    if len(rfds) != n:
                        raise RuntimeError(f"expected {n} descriptors from rank {src}, got {len(rfds)}")
        except Exception as e:  # noqa: BLE001
            error = error or e
        finally:
            if srv is not None:
                srv.close()
        dist.barrier(group=self.group)
        if error is not None:
            for fl in got.values():
                for fd in fl:
                    try:
                        os.close(fd)
                    except OSError:
                        pass
            raise error
        if len(got) != self.world - 1:
            raise RuntimeError(f"received descriptors from {len(got)} of {self.world - 1} peers")
        return got

    def _init_vmm(self, required: bool) -> bool:
        """Build the heap from VMM allocations bound to one multicast object. Returns False (after every rank agreed
        to) when that is not possible here and ``required`` is False."""
        import uuid

        import torch.distributed as dist

        lib = _lib.load()
        ull, vp, ci = ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_int

        def fail_or_fallback(why: str) -> bool:
            if required:
                raise RuntimeError(f"multicast heap not available: {why}")
            return False

        vmm, mc = ci(), ci()
        have = hasattr(lib, "slime_vmm_support") and lib.slime_vmm_support(ctypes.byref(vmm), ctypes.byref(mc)) == 0 and vmm.value and mc.value
        if not self._all_agree(bool(have)):
            return fail_or_fallback("a rank's GPU lacks VMM file-descriptor export or multicast support")
        tags = [None] * self.world
        dist.all_gather_object(tags, uuid.uuid4().hex[:12] if self.rank == 0 else None, group=self.group)
        tag = tags[0]
        st = {"bytes": 0, "gran": 0, "local": 0, "peers": {}, "mc": 0, "mc_va": 0, "bound": False, "fds": []}
        self._vmm = st
        ok = True
        why = ""
        try:
            size, gran = ull(), ull()
            _lib.call("slime_vmm_round_size", ull(self.nbytes), self.world, 1, ctypes.byref(size), ctypes.byref(gran))
            st["bytes"], st["gran"] = size.value, gran.value
            h, va, fd = ull(), vp(), ci()
            _lib.call("slime_vmm_create", ull(st["bytes"]), ull(st["gran"]), ctypes.byref(h), ctypes.byref(va), ctypes.byref(fd))
            st["local"], st["local_va"] = h.value, va.value
            st["fds"].append(fd.value)
            send = [fd.value]
            if self.rank == 0:
                mch, mfd = ull(), ci()
                _lib.call("slime_vmm_mc_create", self.world, ull(st["bytes"]), ctypes.byref(mch), ctypes.byref(mfd))
                st["mc"] = mch.value
                st["fds"].append(mfd.value)
                send.append(mfd.value)
        except Exception as e:  # noqa: BLE001
            ok, why = False, str(e)
            send = []
        if not self._all_agree(ok):
            self._teardown_vmm()
            return fail_or_fallback(why or "another rank could not create its region or the multicast object")
        try:
            got = self._exchange_fds(tag, send)
            for r, fds in got.items():
                st["fds"] += fds
                h, va = ull(), vp()
                _lib.call("slime_vmm_import", fds[0], ull(st["bytes"]), ull(st["gran"]), ctypes.byref(h), ctypes.byref(va))
                st["peers"][r] = (h.value, va.value)
                if r == 0 and self.rank != 0:
                    mch = ull()
                    _lib.call("slime_vmm_mc_import", fds[1], ctypes.byref(mch))
                    st["mc"] = mch.value
            _lib.call("slime_vmm_mc_add_device", ull(st["mc"]))
        except Exception as e:  # noqa: BLE001
            ok, why = False, str(e)
        if not self._all_agree(ok):  # nobody has bound anything yet: safe to back out
            self._teardown_vmm()
            return fail_or_fallback(why or "another rank could not map its peers or join the multicast object")
        try:
            mva = vp()
            _lib.call("slime_vmm_mc_bind_map", ull(st["mc"]), ull(st["local"]), ull(st["bytes"]), ull(st["gran"]), ctypes.byref(mva))
            st["mc_va"], st["bound"] = mva.value, True
        except Exception as e:  # noqa: BLE001
            ok, why = False, str(e)
        if not self._all_agree(ok):
            self._teardown_vmm()
            return fail_or_fallback(why or "another rank could not bind its region to the multicast object")
        for fd in st["fds"]:  # the driver holds its own references now
            try:
                os.close(fd)
            except OSError:
                pass
        st["fds"] = []
        self.nbytes = st["bytes"]
        self.local_ptr = st["local_va"]
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        for r, (_h, va) in st["peers"].items():
            self.peer_ptrs[r] = va
        self.mc_ptr = st["mc_va"]
        _OPEN_VMM_HEAPS.add(self)
        dist.barrier(group=self.group)
        return True

    def _teardown_vmm(self) -> None:
        """Unmap the multicast mapping, unbind, release; then the peers; then this rank's region. Safe to call on a
        partly built heap and more than once."""
        st, self._vmm = self._vmm, None
        if not st:
            return
        ull, vp = ctypes.c_ulonglong, ctypes.c_void_p
        lib = _lib.load()
        if st.get("mc"):
            lib.slime_vmm_mc_teardown(ull(st["mc"]), vp(st.get("mc_va") or None), ull(st["bytes"]), int(bool(st.get("bound"))))
        for _r, (h, va) in st.get("peers", {}).items():
            lib.slime_vmm_unmap_release(ull(h), vp(va), ull(st["bytes"]))
        if st.get("local"):
            lib.slime_vmm_unmap_release(ull(st["local"]), vp(st.get("local_va") or None), ull(st["bytes"]))
        for fd in st.get("fds", []):
            try:
                os.close(fd)
            except OSError:
                pass
        self.mc_ptr = 0
        _OPEN_VMM_HEAPS.discard(self)

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
        for p in (self._owned or ([self.local_ptr] if self._vmm else [])):
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
        if self._vmm is not None:
            self._teardown_vmm()
            return
        for p in self._opened:
            _lib.call("slime_ipc_close", ctypes.c_void_p(p))
        self._opened.clear()
        for p in self._owned:
            _lib.call("slime_symm_free", ctypes.c_void_p(p))
        self._owned.clear()

    def __del__(self):
        try:
            if self._owned or self._opened or self._vmm is not None:
                self.close()
        except Exception:
            pass


# Multicast heaps that are still open; closed at interpreter exit, before CUDA tears the context down, so that no
# rank leaves while its memory is bound to a multicast object.
class _HeapSet:
    def __init__(self):
        self._items: dict[int, "SymmetricHeap"] = {}

    def add(self, h):
        self._items[id(h)] = h

    def discard(self, h):
        self._items.pop(id(h), None)

    def close_all(self):
        for h in list(self._items.values()):
            try:
                h.close()
            except Exception:
                pass


_OPEN_VMM_HEAPS = _HeapSet()

import atexit  # noqa: E402

atexit.register(_OPEN_VMM_HEAPS.close_all)
