"""Low-latency all-gather buffer (``csrc/kernels/allgather.cu``).

Follows the buffer pattern of the reference's removed ``AllGatherInterLLBuffer``
(``dlslime/csrc/python/bind.cpp:533-541`` in the reference): the object owns a
pre-registered symmetric buffer, ``buffer_info()`` is exchanged out of band,
``connect_full_mesh(infos)`` maps the peers, ``all_gather_ll(x)`` gathers, and
``all_gather_ll_hook(x)`` issues the transfer and returns a hook that completes it.
Constructor arguments here: ``(max_bs, msg_size, dtype, world_size, rank)``.
"""

from __future__ import annotations

import ctypes
import struct

import torch

from .. import _lib
from ..parallel.symm import SymmetricHeap
from ._common import default_status, ptr, stream_ptr

_v, _i, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
_lib.declare("slime_ag_push", [ctypes.c_char_p, _v, _ull, _ull, _ull, _v, _i, _i, _v, _v])
_lib.declare("slime_ag_wait", [ctypes.c_char_p, _ull, _v, _v])
_CFG_FMT = "<2i3Q8QQQQ"


class AllGatherLLBuffer:
    def __init__(self, max_bs: int, msg_size: int, dtype: torch.dtype, world_size: int | None = None,
                 rank: int | None = None, *, group=None, heap: SymmetricHeap | None = None, base_off: int | None = None,
                 wait_ns: int = 0, multicast: bool | None = None):
        self.dtype, self.msg_size, self.max_bs = dtype, msg_size, max_bs
        self.itemsize = torch.empty((), dtype=dtype).element_size()
        self.slot_bytes = (max_bs * msg_size * self.itemsize + 255) // 256 * 256
        world = world_size if world_size is not None else (heap.world if heap else None)
        if heap is None:
            import torch.distributed as dist

            world = dist.get_world_size(group) if dist.is_initialized() else 1
            # multicast=None: a multicast-capable heap where the group's GPUs offer one, else plain peer pointers
            heap = SymmetricHeap(2 * world * self.slot_bytes + 4096, group=group, multicast=multicast)
        self.heap, self.world = heap, heap.world
        self.use_multicast = bool(getattr(heap, "mc_ptr", 0)) and multicast is not False
        # Which calls go through the multicast mapping. A multimem store leaves the GPU once instead of once per peer,
        # but the switch also delivers it to the sender's own region, over the sender's own links: small messages,
        # which are bound by the number of stores issued, win; large ones, which are bound by what every rank has to
        # receive, pay world / (world - 1) and lose. SLIME_AG_MULTICAST = always | never | auto (default: groups of
        # four or more ranks, contributions up to SLIME_AG_MULTICAST_MAX_BYTES = 4 MiB).
        import os

        self._mc_policy = os.environ.get("SLIME_AG_MULTICAST", "auto")
        self._mc_max_bytes = int(os.environ.get("SLIME_AG_MULTICAST_MAX_BYTES", str(4 << 20)))
        self.rank = heap.rank if rank is None else rank
        assert world is None or world == self.world
        total = 2 * self.world * self.slot_bytes + 4096
        self.base_off = heap.reserve(total) if base_off is None else base_off
        self.off_data = self.base_off
        self.off_flags = self.base_off + 2 * self.world * self.slot_bytes
        self.step = 0
        # Device-resident step counter: the kernels read and advance it themselves, so calls can be captured in
        # a CUDA graph and replayed. ``self.step`` mirrors it on the host for the view bookkeeping.
        self.step_dev = torch.zeros(1, dtype=torch.int64, device="cuda")
        self.wait_ns = wait_ns
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._counter_ptr = self.counter.data_ptr()
        self.status = default_status()
        self._cfg = self._pack(False)
        self._cfg_mc = self._pack(True) if self.use_multicast else None
        self._views: dict = {}

    def _pack(self, with_mc: bool = False) -> bytes:
        peers = list(self.heap.peer_ptrs) + [0] * (8 - self.world)
        mc = getattr(self.heap, "mc_ptr", 0) if (with_mc and self.use_multicast) else 0
        return struct.pack(_CFG_FMT, self.rank, self.world, self.off_data, self.off_flags, self.slot_bytes, *peers, self.wait_ns,
                           self.step_dev.data_ptr(), mc)

    @classmethod
    def emulated_group(cls, world: int, max_bs: int, msg_size: int, dtype: torch.dtype, wait_ns: int = 0):
        slot = (max_bs * msg_size * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        heap = SymmetricHeap.emulated(world, 2 * world * slot + 4096)
        off = heap.reserve(2 * world * slot + 4096)
        return [cls(max_bs, msg_size, dtype, heap=heap, rank=r, base_off=off, wait_ns=wait_ns) for r in range(world)]

    def buffer_info(self) -> dict:
        return self.heap.export_info()

    def connect_full_mesh(self, infos) -> None:
        self.heap.connect(infos)
        self._cfg = self._pack(False)

    def get_local_buffer(self) -> torch.Tensor:
        return self.heap.view(self.off_data, (2, self.world, self.slot_bytes), torch.uint8, rank=self.rank)

    def _result(self, step: int, bs: int) -> torch.Tensor:
        half = step & 1
        v = self._views.get((half, bs))
        if v is None:  # building a tensor over raw memory is slow; the handful of shapes in use are kept
            off = self.off_data + half * self.world * self.slot_bytes
            v = self._views[(half, bs)] = self.heap.view(off, (self.world * bs, self.msg_size), self.dtype, rank=self.rank)
        return v

    def _issue(self, x: torch.Tensor, do_wait: bool, max_blocks: int = 0) -> tuple[int, int]:
        if not (x.is_contiguous() and x.dtype == self.dtype and x.shape[-1] == self.msg_size):
            raise ValueError("all_gather_ll needs a contiguous [bs, msg_size] tensor of the buffer's dtype")
        bs = x.numel() // self.msg_size
        if bs > self.max_bs:
            raise ValueError(f"batch of {bs} exceeds max_bs={self.max_bs}")
        self.step += 1
        nbytes = x.numel() * self.itemsize
        cfg = self._cfg_mc if self._through_multicast(nbytes) else self._cfg
        _lib.call("slime_ag_push", cfg, x.data_ptr(), nbytes, nbytes, 1, self._counter_ptr, int(do_wait),
                  max_blocks, self.status.dev_ptr, torch.cuda.current_stream().cuda_stream)
        return self.step, bs

    def _through_multicast(self, nbytes: int) -> bool:
        if self._cfg_mc is None or self._mc_policy == "never":
            return False
        if self._mc_policy == "always":
            return True
        return self.world >= 4 and nbytes <= self._mc_max_bytes

    def all_gather_ll(self, x: torch.Tensor) -> torch.Tensor:
        """Gather ``x`` [bs, msg_size] from every rank -> [world * bs, msg_size] (a view of the buffer).

        The view stays valid until the second-next call on this buffer. ``bs`` must be the
        same on every rank.
        """
        step, bs = self._issue(x, do_wait=True)
        return self._result(step, bs)

    def all_gather_ll_hook(self, x: torch.Tensor):
        """Issue the push now; the returned hook waits for the peers and yields the gathered view."""
        step, bs = self._issue(x, do_wait=False)

        def hook() -> torch.Tensor:
            _lib.call("slime_ag_wait", self._cfg, 0, self.status.dev_ptr, stream_ptr())
            return self._result(step, bs)

        return hook


# name of the reference's class
AllGatherInterLLBuffer = AllGatherLLBuffer
