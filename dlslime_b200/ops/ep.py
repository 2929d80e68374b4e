"""Expert-parallel dispatch / combine buffers (``csrc/kernels/ep.cu``).

``EpBuffer`` owns the symmetric memory one rank needs for a MoE layer: the count
matrix, the packed fp8 receive buffers with scales and source info, the combine
staging buffer and the flag words. The API follows the buffer pattern of the
reference's removed all-to-all ops (``dlslime/csrc/python/bind.cpp:515-531``:
construct, ``buffer_info()``, ``connect_full_mesh()``, then the low-latency op).
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import torch

from .. import _lib
from ..parallel.symm import SymmetricHeap
from ._common import default_status, ptr, stream_ptr

_CFG_FMT = "<8i8Q8QQQQQ"


@dataclass
class EpLayout:
    off_counts: int
    off_dispatch_done: int
    off_combine_done: int
    off_barrier: int
    off_x: int
    off_scale: int
    off_info: int
    off_combine: int
    off_arrive: int
    total: int


def ep_layout(world: int, num_experts: int, topk: int, hidden: int, max_tokens: int, recv_cap: int) -> EpLayout:
    cur = 0

    def take(n):
        nonlocal cur
        off = (cur + 255) // 256 * 256
        cur = off + n
        return off

    return EpLayout(
        off_counts=take(8 * world * num_experts),
        off_dispatch_done=take(8 * 8),
        off_combine_done=take(8 * 8),
        off_barrier=take(8 * 8),
        off_x=take(recv_cap * hidden),
        off_scale=take(recv_cap * (hidden // 128) * 4),
        off_info=take(recv_cap * 8),
        off_combine=take(max_tokens * topk * hidden * 2),
        off_arrive=take(8 * world * (num_experts // world)),
        total=(cur + 255) // 256 * 256,
    )


class EpBuffer:
    """Per-rank state of the dispatch/combine protocol.

    Parameters
    ----------
    num_experts, topk, hidden : model shape (hidden must be a multiple of 512).
    max_tokens : largest number of tokens this rank dispatches in one step.
    recv_cap : rows of the packed receive buffer; defaults to the worst case
        ``world * max_tokens * min(topk, experts_per_rank)`` so no step can overflow.
    heap : an existing :class:`SymmetricHeap` to carve from (else one is created
        over ``group``).
    """

    def __init__(self, num_experts: int, topk: int, hidden: int, max_tokens: int, *, group=None,
                 recv_cap: int | None = None, heap: SymmetricHeap | None = None, rank: int | None = None,
                 base_off: int | None = None, wait_ns: int = 0):
        if heap is None:
            import torch.distributed as dist

            world = dist.get_world_size(group) if dist.is_initialized() else 1
            epr = num_experts // world
            cap = recv_cap or world * max_tokens * min(topk, epr)
            lay = ep_layout(world, num_experts, topk, hidden, max_tokens, cap)
            heap = SymmetricHeap(lay.total, group=group)
            self._own_heap = True
        else:
            self._own_heap = False
        self.heap = heap
        self.world = heap.world
        self.rank = heap.rank if rank is None else rank
        self.num_experts, self.topk, self.hidden, self.max_tokens = num_experts, topk, hidden, max_tokens
        assert num_experts % self.world == 0 and hidden % 512 == 0 and topk <= 8 and self.world <= 8
        self.experts_per_rank = num_experts // self.world
        self.recv_cap = recv_cap or self.world * max_tokens * min(topk, self.experts_per_rank)
        self.layout = ep_layout(self.world, num_experts, topk, hidden, max_tokens, self.recv_cap)
        self.base_off = heap.reserve(self.layout.total) if base_off is None else base_off
        self.wait_ns = wait_ns
        self.epoch = 0
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        # rank-local scratch
        self.topk_idx = torch.empty((max_tokens, topk), dtype=torch.int32, device=dev)
        self.topk_w = torch.empty((max_tokens, topk), dtype=torch.float32, device=dev)
        self.slot = torch.empty((max_tokens, topk), dtype=torch.int32, device=dev)
        self.send_count = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.block_counters = torch.zeros(4, dtype=torch.int32, device=dev)
        self.group_offsets = torch.zeros(self.experts_per_rank + 1, dtype=torch.int32, device=dev)
        # scratch of the streamed form (rows pushed expert by expert; see route_ordered / dispatch_ordered / recv_dequant_gated)
        self.push_off = torch.zeros(num_experts + 1, dtype=torch.int32, device=dev)
        self.perm = torch.zeros(max_tokens * topk, dtype=torch.int32, device=dev)
        self.xq_stage = self.xs_stage = None  # tokens quantised once per step (allocated on first use)
        # optional timing of the streamed form (enable_stream_trace): when each expert became ready, and when the
        # GEMM's first CTA began to wait for / got each group
        self.ready_time = self.group_trace = None
        self.pushed = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self.deq_done = torch.zeros(self.experts_per_rank, dtype=torch.int32, device=dev)
        self.group_ready = torch.zeros(self.experts_per_rank, dtype=torch.int64, device=dev)
        # Device-resident step counter for graph-replayable steps (methods called with epoch=None use it).
        self.epoch_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        self.trace = None  # device trace page, see enable_device_trace
        self._cfg = self._pack_cfg()
        self._cfg_dev = self._pack_cfg(self.epoch_dev.data_ptr())
        self.status = default_status()
        self._bc0, self._bc1 = self.block_counters[0:].data_ptr(), self.block_counters[1:].data_ptr()

    # -- config ------------------------------------------------------------------
    def _pack_cfg(self, epoch_ptr: int = 0) -> bytes:
        L, b = self.layout, self.base_off
        peers = list(self.heap.peer_ptrs) + [0] * (8 - self.world)
        return struct.pack(
            _CFG_FMT, self.rank, self.world, self.num_experts, self.experts_per_rank, self.topk, self.hidden,
            self.max_tokens, self.recv_cap,
            b + L.off_counts, b + L.off_dispatch_done, b + L.off_combine_done, b + L.off_barrier,
            b + L.off_x, b + L.off_scale, b + L.off_info, b + L.off_combine, *peers, self.wait_ns, epoch_ptr,
            self.trace.data_ptr() if self.trace is not None else 0, b + L.off_arrive)

    # -- device trace ---------------------------------------------------------------
    _TRACE_KERNELS = ("dispatch", "receive", "combine", "wait", "barrier")

    def enable_device_trace(self, on: bool = True) -> None:
        """Let the kernels of this buffer that wait for other ranks record, in device memory, when they last started
        and how long they waited (``globaltimer`` nanoseconds), and let dispatch count the rows it pushes to each
        peer. Costs one predictable branch per kernel when off. A step captured in a CUDA graph before this call keeps
        the setting it was captured with."""
        self.trace = torch.zeros(64, dtype=torch.int64, device=self.epoch_dev.device) if on else None
        self._cfg = self._pack_cfg()
        self._cfg_dev = self._pack_cfg(self.epoch_dev.data_ptr())

    def device_trace(self) -> dict:
        """Snapshot of the trace page (synchronises the device): per kernel ``{calls, last_start_ns, last_wait_ns,
        total_wait_ns}``, and per peer the rows and bytes (fp8 payload + scales + source word) dispatched so far."""
        if self.trace is None:
            raise RuntimeError("device trace is off; call enable_device_trace() first")
        t = self.trace.cpu().view(16, 4).tolist()
        row_bytes = self.hidden + self.hidden // 128 * 4 + 8
        out = {name: dict(zip(("calls", "last_start_ns", "last_wait_ns", "total_wait_ns"), t[i]))
               for i, name in enumerate(self._TRACE_KERNELS)}
        out["peers"] = [{"rank": p, "rows": t[8 + p][0], "bytes": t[8 + p][0] * row_bytes, "steps": t[8 + p][1]}
                        for p in range(self.world)]
        return out

    @classmethod
    def emulated_group(cls, world: int, num_experts: int, topk: int, hidden: int, max_tokens: int,
                       recv_cap: int | None = None, wait_ns: int = 0) -> list["EpBuffer"]:
        """``world`` buffers on ONE device that address each other like ranks on separate GPUs.

        Meant for single-GPU tests: run each protocol step for every rank before the next
        step, so that every wait finds its flag already published.
        """
        epr = num_experts // world
        cap = recv_cap or world * max_tokens * min(topk, epr)
        lay = ep_layout(world, num_experts, topk, hidden, max_tokens, cap)
        heap = SymmetricHeap.emulated(world, lay.total)
        off = heap.reserve(lay.total)
        return [cls(num_experts, topk, hidden, max_tokens, recv_cap=cap, heap=heap, rank=r, base_off=off, wait_ns=wait_ns)
                for r in range(world)]

    def buffer_info(self) -> dict:
        return self.heap.export_info()

    def connect_full_mesh(self, infos) -> None:
        self.heap.connect(infos)
        self._cfg = self._pack_cfg()
        self._cfg_dev = self._pack_cfg(self.epoch_dev.data_ptr())

    # -- views into this rank's region ----------------------------------------------
    def _view(self, off, shape, dtype):
        return self.heap.view(self.base_off + off, shape, dtype, rank=self.rank)

    @property
    def recv_x(self) -> torch.Tensor:
        return self._view(self.layout.off_x, (self.recv_cap, self.hidden), torch.float8_e4m3fn)

    @property
    def recv_scale(self) -> torch.Tensor:
        return self._view(self.layout.off_scale, (self.recv_cap, self.hidden // 128), torch.float32)

    @property
    def recv_info(self) -> torch.Tensor:
        return self._view(self.layout.off_info, (self.recv_cap,), torch.int64)

    @property
    def combine_buf(self) -> torch.Tensor:
        return self._view(self.layout.off_combine, (self.max_tokens * self.topk, self.hidden), torch.bfloat16)

    def scatter_bases(self):
        """Base address of every rank's combine buffer (for the GEMM scatter epilogue)."""
        import ctypes

        arr = (ctypes.c_ulonglong * 8)()
        for r in range(self.world):
            arr[r] = self.heap.peer_ptrs[r] + self.base_off + self.layout.off_combine
        return arr

    # -- protocol steps -----------------------------------------------------------------
    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # Every step method takes ``epoch``: an explicit step number (the caller counts), or None to use the
    # device-resident counter, which route() advances; the latter form can be captured in a CUDA graph.
    def _mode(self, epoch, first: bool = False):
        return (self._cfg_dev, 1 if first else 0) if epoch is None else (self._cfg, epoch)

    def route(self, logits: torch.Tensor | None, T: int, epoch: int | None = None, renormalize: bool = False) -> None:
        """Top-k routing (or counting of caller-provided ``topk_idx``) and count broadcast."""
        cfg, e = self._mode(epoch, first=True)
        _lib.call("slime_ep_route", cfg, ptr(logits), T, ptr(self.topk_idx), ptr(self.topk_w), ptr(self.slot),
                  ptr(self.send_count), self._bc0, e, int(renormalize), stream_ptr())

    def dispatch(self, x: torch.Tensor, epoch: int | None = None, max_blocks: int = 0) -> None:
        """Quantise ``x`` [T, hidden] bf16 to fp8 and push every (token, expert) copy to its owner."""
        T = x.shape[0]
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] == self.hidden
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_dispatch", cfg, ptr(x), x.stride(0), T, ptr(self.topk_idx), ptr(self.slot),
                  ptr(self.group_offsets), self._bc1, e, max_blocks,
                  self.status.dev_ptr, stream_ptr())

    # -- streamed form ------------------------------------------------------------------
    def route_ordered(self, logits: torch.Tensor | None, T: int, epoch: int | None = None, renormalize: bool = False) -> None:
        """``route`` that also lays out this rank's push order (expert by expert) for ``dispatch_ordered``."""
        cfg, e = self._mode(epoch, first=True)
        _lib.call("slime_ep_route_ordered", cfg, ptr(logits), T, ptr(self.topk_idx), ptr(self.topk_w), ptr(self.slot),
                  ptr(self.send_count), self._bc0, e, int(renormalize), ptr(self.push_off), stream_ptr())

    def compute_layout(self, epoch: int | None = None) -> None:
        """One block that waits for every rank's counts and writes ``group_offsets``; lets the kernels that walk the
        expert groups be launched without waiting for the dispatch kernel."""
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_layout", cfg, ptr(self.group_offsets), e, self.status.dev_ptr, stream_ptr())

    def dispatch_ordered(self, x: torch.Tensor, epoch: int | None = None, max_blocks: int = 0) -> None:
        """Quantise and push every (token, expert) row in push order; each completed (destination, expert) publishes
        an arrival word on the destination."""
        T = self._stage_quantised(x)
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_dispatch_ordered", cfg, ptr(self.xq_stage), ptr(self.xs_stage), T, ptr(self.topk_idx), ptr(self.slot),
                  ptr(self.push_off), ptr(self.perm), ptr(self.pushed), e, max_blocks, self.status.dev_ptr, stream_ptr())

    def _stage_quantised(self, x: torch.Tensor) -> int:
        T = x.shape[0]
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] == self.hidden
        if self.xq_stage is None:
            self.xq_stage = torch.empty((self.max_tokens, self.hidden), dtype=torch.float8_e4m3fn, device=self.device)
            self.xs_stage = torch.empty((self.max_tokens, self.hidden // 128), dtype=torch.float32, device=self.device)
        # every token is quantised once, here; the push then only copies rows
        _lib.call("slime_fp8_quant_1x128", ptr(x), ptr(self.xq_stage), ptr(self.xs_stage), T, self.hidden, x.stride(0),
                  self.hidden, stream_ptr())
        return T

    def stage_quantised(self, x: torch.Tensor) -> None:
        """Quantise this step's tokens into the local staging buffer (independent of routing, so it can run first)."""
        self._stage_quantised(x)

    def stream_comm(self, T: int, out: torch.Tensor, epoch: int | None = None, blocks: int = 0) -> None:
        """Ordered push of the staged rows and gated receive into ``out`` as ONE kernel (two pushing blocks and one
        receiving block per SM). The gated grouped GEMM launched next on the same stream starts beside it."""
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_stream_comm", cfg, ptr(self.xq_stage), ptr(self.xs_stage), T, ptr(self.topk_idx), ptr(self.slot),
                  ptr(self.push_off), ptr(self.perm), ptr(self.pushed), ptr(self.group_offsets), ptr(out), out.stride(0),
                  ptr(self.deq_done), ptr(self.group_ready), ptr(self.ready_time), e, blocks, self.status.dev_ptr, stream_ptr())

    def recv_dequant_gated(self, out: torch.Tensor, epoch: int | None = None, max_blocks: int = 0) -> None:
        """Per local expert: wait for its rows from every rank, expand them to bf16 ``out``, publish
        ``group_ready[j]`` = step for the gated grouped GEMM."""
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_recv_dequant_gated_traced", cfg, ptr(self.group_offsets), ptr(out), out.stride(0), ptr(self.deq_done),
                  ptr(self.group_ready), ptr(self.ready_time), e, max_blocks, self.status.dev_ptr, stream_ptr())

    def enable_stream_trace(self, on: bool = True) -> None:
        """Record, in device memory, when the gated receive published each expert (``ready_time`` [experts_per_rank],
        ``globaltimer`` ns) and when the first CTA of the gated GEMM began to wait for and obtained each group
        (``group_trace`` [experts_per_rank, 2]). Shows which of the two kernels waits for the other."""
        epr = self.experts_per_rank
        self.ready_time = torch.zeros(epr, dtype=torch.int64, device=self.device) if on else None
        # [epr, 2] wait-start / ready per group, then one start time per CTA of the GEMM (up to 256 CTAs)
        self.group_trace = torch.zeros(2 * epr + 256, dtype=torch.int64, device=self.device) if on else None

    def recv_dequant(self, out: torch.Tensor, epoch: int | None, expected_rows: int) -> None:
        """Wait for every rank's rows, then expand the packed fp8 rows to bf16 ``out`` [recv_cap, hidden]."""
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_recv_dequant", cfg, ptr(self.group_offsets), ptr(out), out.stride(0), expected_rows,
                  e, self.status.dev_ptr, stream_ptr())

    def combine_push(self, y: torch.Tensor, expected_rows: int) -> None:
        _lib.call("slime_ep_combine_push", self._cfg, ptr(y), y.stride(0), ptr(self.group_offsets), expected_rows,
                  self.status.dev_ptr, stream_ptr())

    def signal(self, which: int, epoch: int | None = None) -> None:
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_signal", cfg, which, e, stream_ptr())

    def wait(self, which: int, epoch: int | None = None) -> None:
        """One small block that waits for every rank's flag (0 dispatch done, 1 combine done) of this step."""
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_wait", cfg, which, e, self.status.dev_ptr, stream_ptr())

    def combine_reduce(self, out: torch.Tensor, T: int, epoch: int | None = None, do_signal: bool = True) -> None:
        cfg, e = self._mode(epoch)
        _lib.call("slime_ep_combine_reduce", cfg, T, ptr(self.topk_idx), ptr(self.topk_w), ptr(out), out.stride(0),
                  e, int(do_signal), self.status.dev_ptr, stream_ptr())

    def barrier(self, epoch: int) -> None:
        _lib.call("slime_ep_barrier", self._cfg, epoch, self.status.dev_ptr, stream_ptr())


_lib.declare("slime_ep_config_size", [])
import ctypes as _ct  # noqa: E402

_v, _i, _ll, _ull = _ct.c_void_p, _ct.c_int, _ct.c_longlong, _ct.c_ulonglong
_lib.declare("slime_ep_route", [_ct.c_char_p, _v, _i, _v, _v, _v, _v, _v, _ull, _i, _v])
_lib.declare("slime_ep_dispatch", [_ct.c_char_p, _v, _ll, _i, _v, _v, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_route_ordered", [_ct.c_char_p, _v, _i, _v, _v, _v, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_layout", [_ct.c_char_p, _v, _ull, _v, _v])
_lib.declare("slime_ep_dispatch_ordered", [_ct.c_char_p, _v, _v, _i, _v, _v, _v, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_recv_dequant_gated", [_ct.c_char_p, _v, _v, _ll, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_stream_comm", [_ct.c_char_p, _v, _v, _i, _v, _v, _v, _v, _v, _v, _v, _ll, _v, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_recv_dequant_gated_traced", [_ct.c_char_p, _v, _v, _ll, _v, _v, _v, _ull, _i, _v, _v])
_lib.declare("slime_ep_recv_dequant", [_ct.c_char_p, _v, _v, _ll, _i, _ull, _v, _v])
_lib.declare("slime_ep_combine_push", [_ct.c_char_p, _v, _ll, _v, _i, _v, _v])
_lib.declare("slime_ep_signal", [_ct.c_char_p, _i, _ull, _v])
_lib.declare("slime_ep_wait", [_ct.c_char_p, _i, _ull, _v, _v])
_lib.declare("slime_ep_combine_reduce", [_ct.c_char_p, _i, _v, _v, _v, _ll, _ull, _i, _v, _v])
_lib.declare("slime_ep_barrier", [_ct.c_char_p, _ull, _v, _v])
