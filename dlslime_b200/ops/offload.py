"""Device <-> pinned host staging on a side stream (the offloading engine).

The reference only sketches this component (``dlslime/csrc/engine/offloading/offloading.h:5-21`` in the
reference lists an Offloader / Loader / DRAM pool as future work). Here: a pinned DRAM pool carved into equal
slots, ``offload`` (HBM -> DRAM) and ``load`` (DRAM -> HBM) as asynchronous copies on a dedicated stream with
events for ordering, and back-pressure when every slot is taken.
"""

from __future__ import annotations

import threading

import torch


class DRAMMemoryPool:
    def __init__(self, slot_bytes: int, num_slots: int):
        self.slot_bytes, self.num_slots = int(slot_bytes), int(num_slots)
        self.buf = torch.empty((num_slots, slot_bytes), dtype=torch.uint8).pin_memory() if torch.cuda.is_available() \
            else torch.empty((num_slots, slot_bytes), dtype=torch.uint8)
        self._free = list(range(num_slots))
        self._cv = threading.Condition()

    def acquire(self, timeout: float | None = None) -> int:
        with self._cv:
            if not self._cv.wait_for(lambda: self._free, timeout):
                raise TimeoutError("no free DRAM slot (back-pressure)")
            return self._free.pop()

    def release(self, slot: int) -> None:
        with self._cv:
            self._free.append(slot)
            self._cv.notify()

    def slot(self, i: int) -> torch.Tensor:
        return self.buf[i]


class Offloader:
    """Asynchronous HBM -> DRAM; returns (slot, event). ``Loader`` brings a slot back."""

    def __init__(self, pool: DRAMMemoryPool):
        self.pool = pool
        self.stream = torch.cuda.Stream()

    def offload(self, t: torch.Tensor, timeout: float | None = None):
        nbytes = t.numel() * t.element_size()
        if nbytes > self.pool.slot_bytes:
            raise ValueError(f"tensor of {nbytes} bytes does not fit a slot of {self.pool.slot_bytes}")
        slot = self.pool.acquire(timeout)
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self.pool.slot(slot)[:nbytes].copy_(t.contiguous().view(torch.uint8).reshape(-1), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        return slot, ev


class Loader:
    def __init__(self, pool: DRAMMemoryPool):
        self.pool = pool
        self.stream = torch.cuda.Stream()

    def load(self, slot: int, out: torch.Tensor, after: "torch.cuda.Event | None" = None, release: bool = True):
        nbytes = out.numel() * out.element_size()
        with torch.cuda.stream(self.stream):
            if after is not None:
                self.stream.wait_event(after)
            out.view(torch.uint8).reshape(-1).copy_(self.pool.slot(slot)[:nbytes], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        if release:
            ev.synchronize()
            self.pool.release(slot)
        return ev
