"""NVLink endpoint: batched one-sided read / write between GPUs of one node.

API parity with the reference's ``NVLinkEndpoint``
(``dlslime/csrc/engine/nvlink/nvlink_endpoint.h:22-113`` in the reference):
``register_memory_region(addr, offset, length, name)``, ``endpoint_info()``,
``connect(info)``, ``read(assign, stream)`` with handle tuples
``(local_handle, remote_handle, remote_offset, local_offset, length)`` or named
tuples ``(local_name, remote_name, remote_offset, local_offset, length)``, and the
same ``mr_info`` JSON (``name, addr, offset, length, ipc_handle[64]``).

Beyond the reference: a whole batch is ONE kernel launch
(``csrc/kernels/nvlink_endpoint.cu``), ``write`` exists, and
``write_with_imm`` / ``imm_recv`` publish and consume a completion word, so the
future returned here really completes (the reference's future is a no-op and its
caller must synchronise the stream).
"""

from __future__ import annotations

import ctypes
import os
import time
from typing import Sequence

import numpy as np
import torch

from .. import _lib
from ._common import stream_ptr

_v, _i, _ull, _cp = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_char_p
_ubp = ctypes.POINTER(ctypes.c_ubyte)
_ullp = ctypes.POINTER(ctypes.c_ulonglong)
_lib.declare("slime_nvlink_ep_destroy", [_v])
_lib.declare("slime_nvlink_ep_register", [_v, _ull, _ull, _cp])
_lib.declare("slime_nvlink_ep_unregister", [_v, _i])
_lib.declare("slime_nvlink_ep_local_info", [_v, _i, _ubp, _ullp, _ullp, _ullp])
_lib.declare("slime_nvlink_ep_register_remote", [_v, _cp, _ubp, _ull, _ull, _ull, _i])
_lib.declare("slime_nvlink_ep_handle", [_v, _cp, _i])
_lib.declare("slime_nvlink_ep_transfer", [_v, _v, _i, _i, _v, _ull, _i, _i, _v])
_lib.declare("slime_nvlink_ep_status", [_v, ctypes.POINTER(ctypes.c_uint)])
_lib.declare("slime_nvlink_ep_status_clear", [_v])
_lib.declare("slime_nvlink_ep_tune", [_i, _i])
_ll = ctypes.c_longlong
_lib.declare("slime_nvlink_ep_copy1", [_v, _ll, _ll, _ull, _ull, _ull, _i, _v, _ull, _v])

IMM_RING = 1024  # immediate values a peer may have outstanding before the receiver consumes them


def tune(unit_kb: int = 0, bulk: int = -1) -> None:
    """Process-wide tuning of the batched transfer kernels: ``unit_kb`` is the work unit CTAs take from a batch (16 ..
    1024 KiB, default 64; smaller units put several CTAs on one piece at the same time), ``bulk`` picks the
    bulk-copy-engine kernel (1) or the load/store kernel (0) for batches that are 16-byte aligned throughout."""
    _lib.call("slime_nvlink_ep_tune", int(unit_kb), int(bulk))


class NVLinkFuture:
    """Completion of one batched transfer.

    ``wait()`` returns 0 once the kernel has published the completion word (a word in
    mapped host memory, so no stream synchronise is needed), or 402 after ``timeout``.
    """

    def __init__(self, flags_host: int | None, index: int, target: int, stream, on_done=None, status=None):
        self._host, self._index, self._target, self._stream = flags_host, index, target, stream
        self._on_done = on_done  # called once, the first time completion is observed (accounting)
        self._status = status  # callable -> kernel status code of the endpoint (non-zero: the word will never come)

    def done(self) -> bool:
        if self._host is None:
            return True
        if ctypes.c_ulonglong.from_address(self._host + 8 * self._index).value < self._target:
            return False
        if self._on_done is not None:
            cb, self._on_done = self._on_done, None
            cb()
        return True

    def wait(self, timeout: float | None = 30.0) -> int:
        if self._host is None:
            return 0
        t0 = time.monotonic()
        polls = 0
        while not self.done():
            polls += 1
            if polls % 64:
                continue  # a tight poll of the mapped word: small transfers complete within microseconds
            now = time.monotonic()
            if timeout is not None and now - t0 > timeout:
                return 402
            if self._status is not None and polls % 4096 == 0 and self._status() != 0:
                return 402  # a copy of this endpoint gave up: its completion word was withheld
            if now - t0 > 200e-6:
                time.sleep(0)  # long transfer: let other threads of the process run between polls
        return 0


class NVLinkEndpoint:
    def __init__(self):
        lib = _lib.load()
        lib.slime_nvlink_ep_create.restype = ctypes.c_void_p
        lib.slime_nvlink_ep_create.argtypes = []
        lib.slime_nvlink_ep_remote_addr.restype = ctypes.c_ulonglong
        lib.slime_nvlink_ep_remote_addr.argtypes = [_v, _i]
        self._h = lib.slime_nvlink_ep_create()
        self._copy1 = lib.slime_nvlink_ep_copy1
        # Accounting (DLSLIME_OBS=1): this endpoint is one link of kind "nvlink" in the process's counters, with the same
        # submit / complete semantics per user operation as the RDMA links. Off: one `is None` test per transfer.
        self._obs_link = None
        from .. import _slime_c

        if _slime_c.obs_enabled():
            self._obs = _slime_c
            self._obs_link = _slime_c.obs_register_link(f"nvlink:gpu{torch.cuda.current_device()}", "nvlink")
        self._names: dict[int, str] = {}
        self._pid = os.getpid()
        self._uid = f"{self._pid}:{id(self):x}"
        # completion words in mapped host memory: slot i belongs to the i-th outstanding transfer
        hp, dp = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.call("slime_host_flags_alloc", 256, ctypes.byref(hp), ctypes.byref(dp))
        self._flags_host, self._flags_dev = hp.value, dp.value
        self._flag_seq = [0] * 256
        self._next_flag = 0
        # imm mailbox: device words that peers write; [0] = producer counter, [1..] ring of values
        self._imm = torch.zeros(IMM_RING + 8, dtype=torch.int64, device="cuda")
        self._imm_read = 0
        self._poll_stream = torch.cuda.Stream()
        self._imm_sent: dict[int, int] = {}
        self.register_memory_region(self._imm.data_ptr(), 0, self._imm.numel() * 8, "sys.imm")

    # -- memory regions -----------------------------------------------------------------
    def register_memory_region(self, addr: int, offset: int, length: int, name: str | None = None) -> int:
        """Register ``[addr + offset, addr + offset + length)``; returns the local handle."""
        h = _lib.call("slime_nvlink_ep_register", self._h, int(addr) + int(offset), int(length),
                      name.encode() if name else None)
        self._names[h] = name or f"auto_0x{int(addr) + int(offset):x}"
        return h

    def unregister_memory_region(self, handle: int) -> int:
        _lib.call("slime_nvlink_ep_unregister", self._h, handle)
        self._names.pop(handle, None)
        return 0

    def get_mr_handle(self, name: str) -> int:
        return _lib.load().slime_nvlink_ep_handle(self._h, name.encode(), 0)

    def get_remote_mr_handle(self, name: str) -> int:
        return _lib.load().slime_nvlink_ep_handle(self._h, name.encode(), 1)

    def mr_info(self) -> dict:
        out = {}
        for h, name in self._names.items():
            ipc = (ctypes.c_ubyte * 64)()
            off, addr, length = _ull(), _ull(), _ull()
            _lib.call("slime_nvlink_ep_local_info", self._h, h, ipc, ctypes.byref(off), ctypes.byref(addr), ctypes.byref(length))
            signed = [b - 256 if b > 127 else b for b in bytes(ipc)]  # the reference serialises the handle as int8
            out[name] = {"name": name, "addr": addr.value, "offset": off.value, "length": length.value,
                         "ipc_handle": signed, "owner": self._uid, "handle": h}
        return out

    def endpoint_info(self) -> dict:
        return {"mr_info": self.mr_info()}

    def register_remote_memory_region(self, mr_info: dict, name: str | None = None) -> int:
        ipc = (ctypes.c_ubyte * 64)(*[int(b) & 0xFF for b in mr_info["ipc_handle"]])
        same = str(mr_info.get("owner", "")).split(":")[0] == str(self._pid)
        return _lib.call("slime_nvlink_ep_register_remote", self._h, (name or mr_info.get("name", "")).encode(), ipc,
                         int(mr_info["offset"]), int(mr_info["length"]), int(mr_info["addr"]), int(same))

    def connect(self, endpoint_info: dict) -> int:
        """Map every region of the peer. Remote handles follow the peer's handle order."""
        items = sorted(endpoint_info["mr_info"].items(), key=lambda kv: kv[1].get("handle", 0))
        for name, info in items:
            self.register_remote_memory_region(info, name)
        self._peer_imm = self.get_remote_mr_handle("sys.imm")
        return 0

    # -- data path --------------------------------------------------------------------------
    def _resolve(self, assign: Sequence[tuple]) -> np.ndarray:
        if len(assign) and isinstance(assign[0][0], str):
            lib = _lib.load()
            rows = []
            for ln, rn, roff, loff, length in assign:
                lh, rh = lib.slime_nvlink_ep_handle(self._h, ln.encode(), 0), lib.slime_nvlink_ep_handle(self._h, rn.encode(), 1)
                if lh < 0 or rh < 0:
                    raise KeyError(f"memory region not found: local={ln!r} remote={rn!r}")
                rows.append((lh, rh, roff, loff, length))
            assign = rows
        for row in assign:
            if min(int(v) for v in row) < 0:
                raise ValueError(f"negative handle, offset or length in assignment {tuple(row)!r}")
        arr = np.ascontiguousarray(np.asarray(assign, dtype=np.uint64).reshape(-1, 5))
        return arr

    def _account(self, op: int, n: int, nbytes: int, fut: "NVLinkFuture") -> None:
        """One submit now; the completion when the future first sees its word (at once if there is no word)."""
        obs, link = self._obs, self._obs_link
        obs.obs_record_submit(link, op, n, nbytes)
        if fut._host is None:
            obs.obs_record_complete(link, op, nbytes)
        else:
            fut._on_done = lambda: obs.obs_record_complete(link, op, nbytes)

    @staticmethod
    def _batch_size(assign) -> tuple[int, int]:
        if isinstance(assign, np.ndarray):
            return int(assign.shape[0]), int(assign.reshape(-1, 5)[:, 4].sum())
        return len(assign), sum(int(a[4]) for a in assign)

    def _transfer(self, assign, is_write: bool, stream, want_future: bool = True, max_blocks: int = 0):
        if self._obs_link is None:
            return self._transfer_impl(assign, is_write, stream, want_future, max_blocks)
        n, nbytes = self._batch_size(assign)
        fut = self._transfer_impl(assign, is_write, stream, want_future, max_blocks)
        self._account(int(is_write), n, nbytes, fut)  # op indices of the counters: 0 read, 1 write, 2 write_with_imm
        return fut

    def _transfer_impl(self, assign, is_write: bool, stream, want_future: bool = True, max_blocks: int = 0):
        sp = stream_ptr() if stream is None else int(getattr(stream, "cuda_stream", stream))
        if type(assign) is list and len(assign) == 1 and type(assign[0][0]) is int and max_blocks == 0:
            # one contiguous piece by handle: scalar arguments, no table, a copy-engine copy
            lh, rh, roff, loff, length = assign[0]
            if roff < 0 or loff < 0 or length < 0:  # ctypes would turn these into offsets near 2^64
                raise ValueError(f"negative offset or length in assignment {tuple(assign[0])!r}")
            flag_dev, seq, fut = None, 0, None
            if want_future:
                i = self._next_flag
                self._next_flag = (i + 1) % 256
                seq = self._flag_seq[i] = self._flag_seq[i] + 1
                flag_dev = self._flags_dev + 8 * i
                fut = NVLinkFuture(self._flags_host, i, seq, sp)
            if self._copy1(self._h, lh, rh, roff, loff, length, int(is_write), flag_dev, seq, sp) < 0:
                msg = _lib.load().slime_last_error()
                raise _lib.SlimeCudaError(f"slime_nvlink_ep_copy1: {msg.decode(errors='replace') if msg else 'unknown error'}")
            return fut if fut is not None else NVLinkFuture(None, 0, 0, sp)
        arr = assign if isinstance(assign, np.ndarray) else self._resolve(assign)
        if want_future:
            i = self._next_flag
            self._next_flag = (self._next_flag + 1) % 256
            self._flag_seq[i] += 1
            flag_dev = self._flags_dev + 8 * i
            _lib.call("slime_nvlink_ep_transfer", self._h, arr.ctypes.data, arr.shape[0], int(is_write), flag_dev,
                      self._flag_seq[i], 0, max_blocks, sp)
            return NVLinkFuture(self._flags_host, i, self._flag_seq[i], sp, status=self._status_code)
        _lib.call("slime_nvlink_ep_transfer", self._h, arr.ctypes.data, arr.shape[0], int(is_write), None, 0, 0, max_blocks, sp)
        return NVLinkFuture(None, 0, 0, sp)

    def kernel_status(self) -> dict:
        """Status page of this endpoint's kernels: ``code`` 0 = ok, 402 = a bounded wait for a copy ran out."""
        out = (ctypes.c_uint * 4)()
        _lib.call("slime_nvlink_ep_status", self._h, out)
        return {"code": out[0], "where": out[1], "block": out[2], "aux": out[3]}

    def _status_code(self) -> int:
        out = (ctypes.c_uint * 4)()
        _lib.load().slime_nvlink_ep_status(self._h, out)
        return out[0]

    def read(self, assign, stream=None, want_future: bool = True):
        """remote -> local for every tuple; one kernel launch for the whole batch."""
        return self._transfer(assign, False, stream, want_future)

    def write(self, assign, stream=None, want_future: bool = True):
        """local -> remote for every tuple; one kernel launch for the whole batch."""
        return self._transfer(assign, True, stream, want_future)

    def write_with_imm(self, assign, imm_data: int = 0, stream=None):
        """``write`` followed, in stream order, by delivery of ``imm_data`` to the peer's ``imm_recv``."""
        fut = self._transfer_impl(assign, True, stream, want_future=False)
        sp = fut._stream
        n = self._imm_sent.get(self._peer_imm, 0)
        base = _lib.load().slime_nvlink_ep_remote_addr(self._h, self._peer_imm)
        _lib.call("slime_signal_flag_kernel", base + 8 * (1 + n % IMM_RING), (int(imm_data) & 0xFFFFFFFF) | (1 << 32), 0, sp)
        _lib.call("slime_signal_flag_kernel", base, 1, 1, sp)
        self._imm_sent[self._peer_imm] = n + 1
        i = self._next_flag
        self._next_flag = (self._next_flag + 1) % 256
        self._flag_seq[i] += 1
        _lib.call("slime_signal_flag_kernel", self._flags_dev + 8 * i, self._flag_seq[i], 0, sp)
        out = NVLinkFuture(self._flags_host, i, self._flag_seq[i], sp)
        if self._obs_link is not None:
            self._account(2, *self._batch_size(assign), out)
        return out

    def imm_recv(self, timeout: float = 30.0) -> tuple[int, int]:
        """Wait for the next immediate value from the connected peer. Returns (status, imm_data)."""
        t0 = time.monotonic()
        while True:
            with torch.cuda.stream(self._poll_stream):  # polling must not queue behind the caller's work
                head = int(self._imm[0].item())
            if head > self._imm_read:
                with torch.cuda.stream(self._poll_stream):
                    v = int(self._imm[1 + self._imm_read % IMM_RING].item())
                self._imm_read += 1
                return 0, v & 0xFFFFFFFF
            if time.monotonic() - t0 > timeout:
                return 402, 0
            time.sleep(0.0002)

    def close(self) -> None:
        if self._h:
            torch.cuda.synchronize()
            _lib.call("slime_nvlink_ep_destroy", self._h)
            self._h = None
            _lib.call("slime_host_flags_free", ctypes.c_void_p(self._flags_host))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
