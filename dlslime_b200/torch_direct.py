"""GPU-direct send / recv for the ``dlslime`` torch.distributed backend.

The reference's backend hands the device pointer and the current CUDA stream straight to its endpoint
(``dlslime/csrc/torch/slime_backend.cpp:124-168`` in the reference; GPUDirect registration in
``dlslime/csrc/engine/rdma/memory_pool.cpp:74``). On one NVSwitch node the equivalent is a copy from the sender's
tensor into the receiver's tensor over NVLink, with no host bounce. ``DirectGroup`` wraps the backend object that moves
host tensors (the C++ ``c10d::Backend`` or the Python ``SlimeProcessGroup``) and takes over CUDA tensors whose peer is
on the same node:

* ``recv(t)``  exports ``t`` (CUDA IPC handle of its allocation + offset) and sends that description to the source
  as a *ready-to-receive* record on a control endpoint; the work completes when the source's *done* record arrives.
* ``send(t)``  completes once the destination's description has arrived, the peer mapping is open (cached per
  allocation), one ``cudaMemcpyAsync`` device-to-device has run behind the producer kernels of ``t`` and has finished,
  and the *done* record is on its way.

Both records travel on a second endpoint per peer, so they never mix with host-tensor payloads. Every ``wait`` drives
the progress of ALL pending operations towards that peer (descriptions that arrived are matched with queued sends in
order), so the usual exchange patterns (``isend`` + ``irecv`` in either order, ``batch_isend_irecv``) cannot wedge on a
rendezvous. A tensor that cannot be exported (an allocation CUDA IPC refuses) is announced as such and moves through
the wrapped backend's staged path instead. Peers on other hosts, and host tensors, always take the wrapped backend.

``SLIME_BACKEND_DIRECT``: ``auto`` (default: CUDA tensors between GPUs of one host that can address each other),
``off`` (always the staged path), ``shm`` (every tensor through the same protocol with POSIX shared memory in place of
CUDA IPC: the form the CPU tests run).
"""

from __future__ import annotations

import collections
import ctypes
import json
import os
import socket
import struct
import threading
import time
from datetime import timedelta

import torch
import torch.distributed as dist

from . import _slime_c

_WORK_BASE = getattr(dist, "_Work", None) or dist.Work
_REC = struct.Struct("<IIQQ64s40x")  # type, flags, nbytes, offset, handle / name  -> 128 bytes
RTR, DONE, RTR_STAGED = 1, 2, 3
assert _REC.size == 128


class _DirectWork(_WORK_BASE):
    def __init__(self, group: "DirectGroup", peer: int, default_timeout: float):
        super().__init__()
        self._group, self._peer, self._default = group, peer, default_timeout
        self._done = False
        self._error: Exception | None = None
        self._inner = None  # a work of the wrapped backend that finishes this one (staged fallback)
        self._after = None  # called once on completion (receive side in shm mode: copy out of the segment)
        self._fut = torch.futures.Future()

    def _finish(self, error: Exception | None = None):
        if self._done:
            return
        if error is None and self._after is not None:
            self._after()
        self._done, self._error = True, error
        if not self._fut.done():
            if error is None:
                self._fut.set_result(None)
            else:
                self._fut.set_exception(error)

    def wait(self, timeout: timedelta | None = None) -> bool:
        secs = timeout.total_seconds() if isinstance(timeout, timedelta) and timeout.total_seconds() > 0 else self._default
        t0 = time.monotonic()
        spins = 0
        while not self._done:
            self._group._progress(self._peer)
            if self._inner is not None and not self._done:
                self._inner.wait(timedelta(seconds=max(0.001, secs - (time.monotonic() - t0))))
                self._finish()
            if self._done:
                break
            if time.monotonic() - t0 > secs:
                raise RuntimeError("dlslime backend: transfer ended with status 402 (timeout)")
            spins += 1
            if spins > 200:
                time.sleep(0.0002)
        if self._error is not None:
            raise self._error
        return True

    def is_completed(self) -> bool:
        if not self._done:
            self._group._progress(self._peer)
        return self._done

    def is_success(self) -> bool:
        return self._done and self._error is None

    def get_future(self):
        return self._fut


class _Peer:
    def __init__(self):
        self.ctl = None
        self.rx_buf = ctypes.create_string_buffer(128)
        self.rx_fut = None
        self.rtr = collections.deque()      # descriptions received, oldest first
        self.done = 0                       # done records received and not yet matched
        self.sends = collections.deque()    # (tensor, work, ready_event) waiting for a description
        self.recvs = collections.deque()    # works waiting for a done record
        self.tx_keep = collections.deque()  # (buffer, future) of control records in flight
        self.direct = False
        self.lock = threading.Lock()


class DirectGroup(dist.ProcessGroup):
    """See the module docstring. ``inner`` moves host tensors and is the fallback for everything else."""

    def __init__(self, inner, store, rank: int, size: int, timeout: timedelta | None = None, bind_host: str = "127.0.0.1",
                 mode: str = "auto"):
        super().__init__(rank, size)
        self._inner, self._rank, self._size, self._mode = inner, rank, size, mode
        self._timeout = (timeout or timedelta(seconds=300)).total_seconds()
        self._peers: dict[int, _Peer] = {}
        self._opened: dict[bytes, int] = {}  # ipc handle -> mapped base
        self._shm_keep: dict[str, object] = {}
        self._copy_stream = None
        self.counters = {"direct_sends": 0, "direct_recvs": 0, "staged_fallbacks": 0}  # for tests and curiosity
        cuda = torch.cuda.is_available()
        me = {"host": socket.gethostname(), "device": torch.cuda.current_device() if cuda else -1, "pid": os.getpid()}
        store.set(f"SLIME_DIRECT_INFO_{rank}", json.dumps(me))
        infos = {p: json.loads(store.get(f"SLIME_DIRECT_INFO_{p}")) for p in range(size) if p != rank}
        for peer, info in infos.items():
            st = _Peer()
            same_host = info["host"] == me["host"]
            if mode == "shm":
                st.direct = same_host
            elif mode == "auto" and cuda and same_host and info["device"] >= 0:
                st.direct = info["device"] == me["device"] or torch.cuda.can_device_access_peer(me["device"], info["device"])
            if st.direct:
                st.ctl = _slime_c.TcpEndpoint(bind_host, 0, 1)
                store.set(f"SLIME_CTL_{rank}_{peer}", json.dumps(st.ctl.endpoint_info()))
            self._peers[peer] = st
        for peer, st in self._peers.items():
            if st.direct:
                st.ctl.connect(json.loads(store.get(f"SLIME_CTL_{peer}_{rank}")))
                self._post_rx(st)

    def getBackendName(self) -> str:
        return "dlslime"

    # -- control channel ------------------------------------------------------------------------------------------------
    def _post_rx(self, st: _Peer) -> None:
        st.rx_fut = st.ctl.recv((ctypes.addressof(st.rx_buf), 0, 128))

    def _send_record(self, st: _Peer, kind: int, nbytes: int = 0, offset: int = 0, handle: bytes = b"") -> None:
        buf = ctypes.create_string_buffer(_REC.pack(kind, 0, nbytes, offset, handle), 128)
        st.tx_keep.append((buf, st.ctl.send((ctypes.addressof(buf), 0, 128))))
        while len(st.tx_keep) > 64 and st.tx_keep[0][1].done():
            st.tx_keep.popleft()

    # -- export / copy: CUDA IPC, or shared memory in the test mode ------------------------------------------------------
    def _export(self, t: torch.Tensor, work: _DirectWork):
        nbytes = t.numel() * t.element_size()
        if self._mode == "shm":
            from multiprocessing import shared_memory

            seg = shared_memory.SharedMemory(create=True, size=max(nbytes, 1))
            self._shm_keep[seg.name] = seg

            def copy_out(seg=seg, t=t, nbytes=nbytes):
                flat = torch.frombuffer(seg.buf, dtype=torch.uint8, count=nbytes) if nbytes else None
                if nbytes:
                    t.view(-1).view(torch.uint8).copy_(flat)
                del flat
                self._shm_keep.pop(seg.name, None)
                seg.close()
                seg.unlink()

            work._after = copy_out
            return nbytes, 0, seg.name.encode()
        from . import _lib

        h = (ctypes.c_ubyte * 64)()
        off = ctypes.c_ulonglong()
        lib = _lib.load()
        if lib.slime_ipc_get_handle(ctypes.c_void_p(t.data_ptr()), h, ctypes.byref(off), None) != 0:
            return None
        return nbytes, off.value, bytes(h)

    def _copy(self, desc, t: torch.Tensor, ready_event) -> None:
        nbytes, offset, handle = desc
        if nbytes != t.numel() * t.element_size():
            raise RuntimeError(f"dlslime backend: the receiver expects {nbytes} bytes, the sender has {t.numel() * t.element_size()}")
        if self._mode == "shm":
            from multiprocessing import shared_memory

            seg = shared_memory.SharedMemory(name=handle.rstrip(b"\0").decode())
            try:
                if nbytes:
                    dst = torch.frombuffer(seg.buf, dtype=torch.uint8, count=nbytes)
                    dst.copy_(t.contiguous().view(-1).view(torch.uint8))
                    del dst  # the segment cannot be closed while a tensor still exports its buffer
            finally:
                seg.close()
            return
        from . import _lib

        base = self._opened.get(handle)
        if base is None:
            p = ctypes.c_void_p()
            _lib.call("slime_ipc_open", (ctypes.c_ubyte * 64)(*handle), ctypes.byref(p))
            base = self._opened[handle] = p.value
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
        s = self._copy_stream
        s.wait_event(ready_event)  # behind the kernels that produced the tensor
        _lib.call("slime_memcpy_async", ctypes.c_void_p(base + offset), ctypes.c_void_p(t.data_ptr()), ctypes.c_ulonglong(nbytes),
                  ctypes.c_void_p(s.cuda_stream))
        s.synchronize()  # the bytes are in the receiver's memory before it is told so

    # -- progress --------------------------------------------------------------------------------------------------------
    def _progress(self, peer: int) -> None:
        st = self._peers[peer]
        if not st.direct:
            return
        with st.lock:
            while st.rx_fut is not None and st.rx_fut.done():
                status = st.rx_fut.wait(0.0)
                if status != 0:
                    err = RuntimeError(f"dlslime backend: control channel to rank {peer} ended with status {status}")
                    for _t, w, _e in st.sends:
                        w._finish(err)
                    for w in st.recvs:
                        w._finish(err)
                    st.sends.clear()
                    st.recvs.clear()
                    st.rx_fut = None
                    return
                kind, _flags, nbytes, offset, handle = _REC.unpack(st.rx_buf.raw)
                if kind in (RTR, RTR_STAGED):
                    st.rtr.append((kind, nbytes, offset, handle))
                elif kind == DONE:
                    st.done += 1
                self._post_rx(st)
            while st.rtr and st.sends:
                kind, nbytes, offset, handle = st.rtr.popleft()
                t, work, ev = st.sends.popleft()
                if kind == RTR_STAGED:
                    self.counters["staged_fallbacks"] += 1
                    work._inner = self._inner.send([t], peer, 0)
                    continue
                try:
                    self._copy((nbytes, offset, handle), t, ev)
                    self._send_record(st, DONE)
                    self.counters["direct_sends"] += 1
                    work._finish()
                except Exception as e:  # noqa: BLE001
                    work._finish(e)
            while st.done and st.recvs:
                st.done -= 1
                st.recvs.popleft()._finish()

    # -- point to point ------------------------------------------------------------------------------------------------------
    def _direct(self, t: torch.Tensor, peer: int) -> bool:
        st = self._peers.get(peer)
        return st is not None and st.direct and (self._mode == "shm" or t.is_cuda)

    def send(self, tensors, dst: int, tag: int = 0):
        if not all(self._direct(t, dst) for t in tensors):
            return self._inner.send(tensors, dst, tag)
        st, works = self._peers[dst], []
        for t in tensors:
            if not t.is_contiguous():
                raise ValueError("dlslime backend: tensors must be contiguous")
            w = _DirectWork(self, dst, self._timeout)
            ev = None
            if t.is_cuda:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
            with st.lock:
                st.sends.append((t, w, ev))
            works.append(w)
        self._progress(dst)
        return works[0] if len(works) == 1 else _Joined(works)

    def recv(self, tensors, src: int, tag: int = 0):
        if not all(self._direct(t, src) for t in tensors):
            return self._inner.recv(tensors, src, tag)
        st, works = self._peers[src], []
        for t in tensors:
            if not t.is_contiguous():
                raise ValueError("dlslime backend: tensors must be contiguous")
            w = _DirectWork(self, src, self._timeout)
            if t.is_cuda:
                torch.cuda.current_stream().synchronize()  # earlier users of the buffer are done before a peer may write it
            desc = self._export(t, w)
            with st.lock:
                if desc is None:  # not exportable: both sides take the staged path for this tensor
                    self._send_record(st, RTR_STAGED, t.numel() * t.element_size())
                    self.counters["staged_fallbacks"] += 1
                    w._inner = self._inner.recv([t], src, tag)
                else:
                    self._send_record(st, RTR, *desc)
                    self.counters["direct_recvs"] += 1
                    st.recvs.append(w)
            works.append(w)
        self._progress(src)
        return works[0] if len(works) == 1 else _Joined(works)

    def recv_anysource(self, tensors, tag: int = 0):
        raise NotImplementedError("dlslime backend: recv from any source is not supported")

    # -- everything else is the wrapped backend's (collectives raise there) ------------------------------------------------------
    def __getattr__(self, name):
        return getattr(self.__dict__["_inner"], name)

    def _unsupported(self, name):
        raise NotImplementedError(f"dlslime backend: {name} is not supported; it provides send / recv only")

    def broadcast(self, *a, **k):
        self._unsupported("broadcast")

    def allreduce(self, *a, **k):
        self._unsupported("allreduce")

    def allgather(self, *a, **k):
        self._unsupported("allgather")

    def _allgather_base(self, *a, **k):
        self._unsupported("all_gather_into_tensor")

    def reduce_scatter(self, *a, **k):
        self._unsupported("reduce_scatter")

    def alltoall(self, *a, **k):
        self._unsupported("alltoall")

    def alltoall_base(self, *a, **k):
        self._unsupported("all_to_all_single")

    def gather(self, *a, **k):
        self._unsupported("gather")

    def scatter(self, *a, **k):
        self._unsupported("scatter")

    def reduce(self, *a, **k):
        self._unsupported("reduce")

    def barrier(self, *a, **k):
        self._unsupported("barrier")

    def shutdown(self):
        for st in self._peers.values():
            if st.ctl is not None:
                st.ctl.shutdown()
                st.ctl = None
        if self._opened:
            from . import _lib

            for base in self._opened.values():
                _lib.load().slime_ipc_close(ctypes.c_void_p(base))
            self._opened.clear()
        sh = getattr(self._inner, "shutdown", None)
        if callable(sh):
            sh()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


class _Joined(_WORK_BASE):
    """Several works of one call (a tensor list) behind one handle."""

    def __init__(self, works):
        super().__init__()
        self._works = works

    def wait(self, timeout: timedelta | None = None) -> bool:
        for w in self._works:
            w.wait(timeout)
        return True

    def is_completed(self) -> bool:
        return all(w.is_completed() for w in self._works)

    def is_success(self) -> bool:
        return all(w.is_success() for w in self._works)

    def get_future(self):
        return self._works[-1].get_future()
