"""Prefill -> decode KV-cache hand-off for PD-disaggregated serving.

The decode rank owns a paged KV cache inside a symmetric region; its prefill partner
maps that region and, layer by layer, runs ONE kernel that reads the freshly computed
K/V rows of the whole batch and stores them page by page at the positions the decode
side's block table assigned (``csrc/kernels/kv_transfer.cu``). After each layer the
kernel publishes ``layer_done[layer] = step`` in the decode rank's memory, so the
decode side may consume layer ``l`` while ``l + 1`` is still in flight. The transfer
runs on its own stream with a capped number of CTAs and overlaps the prefill compute,
which is represented by a chain of bf16 GEMMs on the tensor cores.

Shape defaults follow a Llama-3-8B shard under TP4: 32 layers, 2 of 8 KV heads per
rank, head_dim 128, 64-token pages. The reference describes this use case only in
prose (``README.md:180-199`` in the reference); its data path would be one
``NVLinkEndpoint.read`` call with one copy per page.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import gemm, kv
from ..ops._common import default_status
from ..parallel.symm import SymmetricHeap


@dataclass
class KVShape:
    layers: int = 32
    kv_heads_local: int = 2
    head_dim: int = 128
    page_tokens: int = 64
    dtype: torch.dtype = torch.bfloat16

    @property
    def row(self) -> int:
        return self.kv_heads_local * self.head_dim

    @property
    def row_bytes(self) -> int:
        return self.row * torch.empty((), dtype=self.dtype).element_size()

    @property
    def page_bytes(self) -> int:
        return self.page_tokens * self.row_bytes


class PagedKVCache:
    """``[layers, 2, num_blocks, page_tokens, row]`` inside a symmetric region, plus per-layer done words."""

    def __init__(self, shape: KVShape, num_blocks: int, heap: SymmetricHeap, owner_rank: int, base_off: int | None = None):
        self.shape, self.num_blocks, self.heap, self.owner = shape, num_blocks, heap, owner_rank
        self.plane_bytes = num_blocks * shape.page_bytes
        self.data_bytes = shape.layers * 2 * self.plane_bytes
        total = self.data_bytes + 8 * shape.layers + 256
        self.base_off = heap.reserve(total) if base_off is None else base_off
        self.flags_off = self.base_off + self.data_bytes

    @staticmethod
    def bytes_needed(shape: KVShape, num_blocks: int) -> int:
        return shape.layers * 2 * num_blocks * shape.page_bytes + 8 * shape.layers + 512

    def plane_addr(self, layer: int, plane: int, rank: int | None = None) -> int:
        r = self.owner if rank is None else rank
        return self.heap.peer_ptrs[r] + self.base_off + (layer * 2 + plane) * self.plane_bytes

    def flag_addr(self, layer: int) -> int:
        return self.heap.peer_ptrs[self.owner] + self.flags_off + 8 * layer

    def tensor(self) -> torch.Tensor:
        s = self.shape
        return self.heap.view(self.base_off, (s.layers, 2, self.num_blocks, s.page_tokens, s.row), s.dtype, rank=self.owner)

    def layer_done(self) -> torch.Tensor:
        return self.heap.view(self.flags_off, (self.shape.layers,), torch.int64, rank=self.owner)


class PrefillSender:
    """Prefill side: per-layer push of a batch's KV pages into a decode rank's paged cache."""

    def __init__(self, shape: KVShape, dst_cache: PagedKVCache, max_tokens: int, comm_blocks: int = 32, comm_threads: int = 256):
        self.shape, self.dst, self.max_tokens = shape, dst_cache, max_tokens
        if comm_threads != 256:
            kv.tune(comm_threads)
        self.kv_stage = torch.empty((shape.layers, 2, max_tokens, shape.row), dtype=shape.dtype, device="cuda")
        self.comm_stream = torch.cuda.Stream(priority=-1)  # transfer CTAs should be placed ahead of the next GEMM's
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.comm_blocks = comm_blocks
        self.step = 0

    def plan(self, prompt_lens, dst_blocks):
        """Upload the page tasks of one batch once; they are reused by every layer."""
        self.tasks = kv.build_page_tasks(prompt_lens, self.shape.page_tokens, dst_blocks)
        self.tokens = int(sum(prompt_lens))
        assert self.tokens <= self.max_tokens
        self.step += 1
        return self.tasks

    def send_layer(self, layer: int, stream=None) -> None:
        tok_off, blk, ntok = self.tasks
        s = self.shape
        kv.kv_move(self.kv_stage[layer, 0].data_ptr(), self.kv_stage[layer, 1].data_ptr(),
                   self.dst.plane_addr(layer, 0), self.dst.plane_addr(layer, 1), tok_off, blk, ntok,
                   page_tokens=s.page_tokens, row_bytes=s.row_bytes, tok_rows=self.max_tokens,
                   page_blocks=self.dst.num_blocks, to_paged=True, done_flag=self.dst.flag_addr(layer),
                   done_value=self.step, counter=self.counter, max_blocks=self.comm_blocks, stream=stream)

    def run_prefill_with_transfer(self, hidden: torch.Tensor, weights: list[torch.Tensor], overlap: bool = True):
        """Synthetic prefill: one [tokens, d] x [d, d] GEMM per layer; layer l's KV goes out while l+1 computes.

        ``hidden`` is ``[tokens, d]`` bf16 and is used as ping-pong scratch with an internal buffer. The
        K/V rows of a layer are taken to be ready in ``kv_stage[layer]`` once that layer's GEMM has run
        (a real model writes them from its attention projections).
        """
        main = torch.cuda.current_stream()
        a, b = hidden, torch.empty_like(hidden)
        for layer in range(self.shape.layers):
            gemm.gemm_bf16(a, weights[layer % len(weights)], out=b)
            a, b = b, a
            if overlap:
                self.comm_stream.wait_stream(main)
                with torch.cuda.stream(self.comm_stream):
                    self.send_layer(layer, self.comm_stream)
            else:
                self.send_layer(layer)
        if overlap:
            main.wait_stream(self.comm_stream)
        return a


def wait_layers(cache: PagedKVCache, step: int, timeout_s: float = 10.0) -> bool:
    """Decode side, host view: True once every layer of ``step`` has landed."""
    import time

    t0 = time.monotonic()
    flags = cache.layer_done()
    while time.monotonic() - t0 < timeout_s:
        if int(flags.min().item()) >= step:
            return True
        time.sleep(0.0005)
    return False
