"""Helpers shared by the op wrappers: stream handles, pointer checks, status pages."""

from __future__ import annotations

import ctypes
import struct
from dataclasses import dataclass

import torch

from .. import _lib

TIME_OUT = 402


def stream_ptr(stream: torch.cuda.Stream | None = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else int(t.data_ptr())


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("this op runs only on CUDA tensors; there is no CPU fallback")


class KernelTimeout(RuntimeError):
    """A bounded device-side wait ran out; the kernel returned without finishing."""

    def __init__(self, info: "StatusInfo"):
        super().__init__(f"device wait timed out: {info}")
        self.info = info
        self.status = TIME_OUT


@dataclass
class StatusInfo:
    code: int
    where: int
    block: int
    aux: int
    expected: int
    observed: int


class StatusPage:
    """32 bytes of mapped pinned host memory that kernels write on a failed wait.

    ``dev_ptr`` is what a kernel receives; ``read()`` needs no copy. The page is
    valid once the stream the kernel ran on has been synchronised.
    """

    _FMT = "<IIIIQQ"

    def __init__(self):
        h, d = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.call("slime_status_alloc", ctypes.byref(h), ctypes.byref(d))
        self.host_ptr, self.dev_ptr = h.value, d.value

    def read(self) -> StatusInfo:
        raw = ctypes.string_at(self.host_ptr, struct.calcsize(self._FMT))
        return StatusInfo(*struct.unpack(self._FMT, raw))

    def clear(self) -> None:
        ctypes.memset(self.host_ptr, 0, struct.calcsize(self._FMT))

    def check(self) -> None:
        info = self.read()
        if info.code != 0:
            self.clear()
            if info.code == TIME_OUT:
                raise KernelTimeout(info)
            raise RuntimeError(f"kernel reported status {info}")

    def close(self) -> None:
        if self.host_ptr:
            _lib.call("slime_status_free", ctypes.c_void_p(self.host_ptr))
            self.host_ptr = self.dev_ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_DEFAULT_STATUS: dict[int, StatusPage] = {}


def default_status() -> StatusPage:
    """One status page per CUDA device, created on first use."""
    dev = torch.cuda.current_device()
    page = _DEFAULT_STATUS.get(dev)
    if page is None:
        page = _DEFAULT_STATUS[dev] = StatusPage()
    return page
