"""Tensor-parallel all-gather -> GEMM over NVLink peer memory.

Every rank holds a shard ``x [rows, K]`` of the activations and a weight shard
``w [N_local, K]``; the result is ``concat_r(x_r) @ w.T``, shape ``[world * rows, N_local]``.
The gathered matrix lives in a symmetric region together with one arrival counter per
128-row chunk. In the fused form (``forward``) ONE kernel does both jobs: extra warps in
every CTA push 32-row slices of the local shard to all ranks and bump the destination's
counters, while the TMA producer of the same kernel waits on the local counters tile by
tile and the tensor-core warps start with the tiles of the local shard. The two-kernel
form (``push`` then ``gemm``) exists for single-GPU replay and as the unfused baseline.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..parallel.symm import SymmetricHeap
from ._common import default_status, ptr, stream_ptr

_v, _i, _ll, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong
_lib.declare("slime_ag_gemm", [_i, _v, _v, _v, _v, _i, _i, _i, _ll, _ll, _i, _i, _v, _v, _ull, _i, _v, _v])


class AllGatherGemm:
    def __init__(self, rows_local: int, k: int, *, group=None, heap: SymmetricHeap | None = None,
                 rank: int | None = None, base_off: int | None = None):
        assert rows_local % 128 == 0 and k % 8 == 0
        if heap is None:
            import torch.distributed as dist

            world = dist.get_world_size(group) if dist.is_initialized() else 1
            heap = SymmetricHeap(self.bytes_needed(rows_local, k, world), group=group)
        self.heap, self.world = heap, heap.world
        self.rank = heap.rank if rank is None else rank
        self.rows_local, self.k = rows_local, k
        self.a_bytes = self.world * rows_local * k * 2
        self.chunks = self.world * rows_local // 128
        total = self.a_bytes + 8 * self.chunks + 256
        self.base_off = heap.reserve(total) if base_off is None else base_off
        self.flags_off = self.base_off + self.a_bytes
        self.step = 0
        self._dst = (ctypes.c_ulonglong * 8)(*[p + self.base_off for p in heap.peer_ptrs], *([0] * (8 - self.world)))
        self._flags = (ctypes.c_ulonglong * 8)(*[p + self.flags_off for p in heap.peer_ptrs], *([0] * (8 - self.world)))
        self.status = default_status()
        self.pair = True  # use the cta_group::2 kernel in forward() when the shard allows it

    @staticmethod
    def bytes_needed(rows_local: int, k: int, world: int) -> int:
        return world * rows_local * k * 2 + 8 * world * rows_local // 128 + 1024

    @classmethod
    def emulated_group(cls, world: int, rows_local: int, k: int):
        heap = SymmetricHeap.emulated(world, cls.bytes_needed(rows_local, k, world))
        off = heap.reserve(cls.bytes_needed(rows_local, k, world) - 512)
        return [cls(rows_local, k, heap=heap, rank=r, base_off=off) for r in range(world)]

    @property
    def gathered(self) -> torch.Tensor:
        return self.heap.view(self.base_off, (self.world * self.rows_local, self.k), torch.bfloat16, rank=self.rank)

    def _call(self, mode, x, w, out, step, push_blocks=0):
        n = w.shape[0] if w is not None else 0
        a_full = self.heap.peer_ptrs[self.rank] + self.base_off
        _lib.call("slime_ag_gemm", mode, ptr(x), a_full, ptr(w), ptr(out), self.rows_local, n, self.k,
                  w.stride(0) if w is not None else self.k, out.stride(0) if out is not None else 0, self.rank, self.world,
                  self._dst, self._flags, step, push_blocks, self.status.dev_ptr, stream_ptr())

    def push(self, x: torch.Tensor, step: int, push_blocks: int = 0) -> None:
        assert x.is_contiguous() and x.shape == (self.rows_local, self.k) and x.dtype == torch.bfloat16
        self._call(0, x, None, None, step, push_blocks)

    def gemm(self, w: torch.Tensor, out: torch.Tensor, step: int) -> None:
        self._call(1, None, w, out, step)

    def forward(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Fused all-gather + GEMM: ``[world * rows, N_local]`` bf16."""
        assert x.is_contiguous() and x.shape == (self.rows_local, self.k) and x.dtype == torch.bfloat16
        assert w.dtype == torch.bfloat16 and w.stride(1) == 1 and w.shape[1] == self.k
        if out is None:
            out = torch.empty((self.world * self.rows_local, w.shape[0]), dtype=torch.bfloat16, device=x.device)
        self.step += 1
        # CTA pairs (256-row tiles) when the shard is a whole number of them
        self._call(3 if self.rows_local % 256 == 0 and self.pair else 2, x, w, out, self.step)
        return out

    __call__ = forward


_lib.declare("slime_ag_gemm_fp8", [_i, _v, _v, _v, _v, _v, _v, _v, _i, _i, _i, _ll, _ll, _i, _i, _v, _v, _v, _ull, _i, _v, _v])


class AllGatherGemmFp8:
    """The same operator with e4m3 activations and weights and DeepSeek-V3 block scales.

    Every rank quantises its shard once (1x128 scales, :func:`dlslime_b200.ops.quant.fp8_quant_1x128`); payload AND
    scales cross NVLink (half the bytes of the bf16 form); the tiles run on the fp8 tensor cores with two-level
    accumulation (``csrc/kernels/common/gemm_fp8.cuh``). The weight shard is quantised ahead of time with 128x128
    scales (``fp8_quant_128x128``). Symmetric layout per rank: gathered payload ``[world * rows, K]`` bytes, gathered
    scales ``[world * rows, K / 128]`` fp32, one arrival counter per 128 rows.
    """

    def __init__(self, rows_local: int, k: int, *, group=None, heap: SymmetricHeap | None = None,
                 rank: int | None = None, base_off: int | None = None):
        assert rows_local % 128 == 0 and k % 128 == 0
        if heap is None:
            import torch.distributed as dist

            world = dist.get_world_size(group) if dist.is_initialized() else 1
            heap = SymmetricHeap(self.bytes_needed(rows_local, k, world), group=group)
        self.heap, self.world = heap, heap.world
        self.rank = heap.rank if rank is None else rank
        self.rows_local, self.k = rows_local, k
        m = self.world * rows_local
        self.a_bytes = m * k
        self.s_bytes = m * (k // 128) * 4
        self.chunks = m // 128
        total = self.a_bytes + self.s_bytes + 8 * self.chunks + 512
        self.base_off = heap.reserve(total) if base_off is None else base_off
        self.s_off = self.base_off + self.a_bytes
        self.flags_off = self.s_off + self.s_bytes
        self.step = 0
        pad = [0] * (8 - self.world)
        self._dst = (ctypes.c_ulonglong * 8)(*[p + self.base_off for p in heap.peer_ptrs], *pad)
        self._sdst = (ctypes.c_ulonglong * 8)(*[p + self.s_off for p in heap.peer_ptrs], *pad)
        self._flags = (ctypes.c_ulonglong * 8)(*[p + self.flags_off for p in heap.peer_ptrs], *pad)
        self.status = default_status()
        self._xq = torch.empty((rows_local, k), dtype=torch.float8_e4m3fn, device="cuda")
        self._sx = torch.empty((rows_local, k // 128), dtype=torch.float32, device="cuda")

    @staticmethod
    def bytes_needed(rows_local: int, k: int, world: int) -> int:
        m = world * rows_local
        return m * k + m * (k // 128) * 4 + 8 * (m // 128) + 2048

    @classmethod
    def emulated_group(cls, world: int, rows_local: int, k: int):
        heap = SymmetricHeap.emulated(world, cls.bytes_needed(rows_local, k, world))
        off = heap.reserve(cls.bytes_needed(rows_local, k, world) - 1024)
        return [cls(rows_local, k, heap=heap, rank=r, base_off=off) for r in range(world)]

    @property
    def gathered(self):
        m = self.world * self.rows_local
        return (self.heap.view(self.base_off, (m, self.k), torch.float8_e4m3fn, rank=self.rank),
                self.heap.view(self.s_off, (m, self.k // 128), torch.float32, rank=self.rank))

    def _call(self, mode, xq, sx, wq, sb, out, step, push_blocks=0):
        n = wq.shape[0] if wq is not None else 0
        base = self.heap.peer_ptrs[self.rank]
        _lib.call("slime_ag_gemm_fp8", mode, ptr(xq), ptr(sx), base + self.base_off, base + self.s_off, ptr(wq), ptr(sb), ptr(out),
                  self.rows_local, n, self.k, wq.stride(0) if wq is not None else self.k, out.stride(0) if out is not None else 0,
                  self.rank, self.world, self._dst, self._sdst, self._flags, step, push_blocks, self.status.dev_ptr, stream_ptr())

    def quantise(self, x: torch.Tensor):
        from . import quant

        assert x.is_contiguous() and x.shape == (self.rows_local, self.k) and x.dtype == torch.bfloat16
        return quant.fp8_quant_1x128(x, self._xq, self._sx)

    def push(self, xq: torch.Tensor, sx: torch.Tensor, step: int, push_blocks: int = 0) -> None:
        self._call(0, xq, sx, None, None, None, step, push_blocks)

    def gemm(self, wq: torch.Tensor, sb: torch.Tensor, out: torch.Tensor, step: int) -> None:
        self._call(1, None, None, wq, sb, out, step)

    def forward(self, x: torch.Tensor, wq: torch.Tensor, sb: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """``x`` bf16 ``[rows, K]`` (quantised here), ``wq`` e4m3 ``[N_local, K]`` with scales ``sb``: ``[world * rows, N_local]`` bf16."""
        assert wq.dtype == torch.float8_e4m3fn and wq.stride(1) == 1 and wq.shape[1] == self.k
        xq, sx = self.quantise(x)
        if out is None:
            out = torch.empty((self.world * self.rows_local, wq.shape[0]), dtype=torch.bfloat16, device=x.device)
        self.step += 1
        self._call(2, xq, sx, wq, sb, out, self.step)
        return out

    __call__ = forward
