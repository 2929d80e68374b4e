"""Paged KV-cache transfer, pack and unpack (``csrc/kernels/kv_transfer.cu``).

Layouts (one rank's shard; ``row = heads_local * head_dim`` elements per token):

* paged cache ``[layers, 2, num_blocks, page_tokens, row]`` -- plane 0 is K, 1 is V;
* token-major staging ``[layers, 2, tokens, row]``.

``build_page_tasks`` turns a batch of prompt lengths plus a destination block table
into flat task arrays (first token row, destination block, rows in the page) that
stay on the device and are reused for every layer.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ._common import default_status, ptr, stream_ptr

_v, _i, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
_lib.declare("slime_kv_transfer", [_ull, _ull, _ull, _ull, _v, _v, _v, _i, _i, _ull, _ull, _ull, _i, _v, _ull, _v, _i, _v, _v])


def build_page_tasks(prompt_lens, page_tokens: int, dst_blocks, src_starts=None, device="cuda"):
    """Flat page tasks for a batch of prompts.

    ``dst_blocks`` lists one destination block per page, prompt after prompt.
    ``src_starts`` gives each prompt's first row on the token-major side (default: packed
    back to back). Returns int32 device tensors ``(tok_off, blk, ntok)``.
    """
    tok_off, ntok = [], []
    start = 0
    for i, n in enumerate(prompt_lens):
        s = start if src_starts is None else src_starts[i]
        for j in range(0, n, page_tokens):
            tok_off.append(s + j)
            ntok.append(min(page_tokens, n - j))
        start += n
    assert len(tok_off) == len(dst_blocks), "one destination block per page is required"
    mk = lambda v: torch.tensor(list(v), dtype=torch.int32, device=device)
    return mk(tok_off), mk(dst_blocks), mk(ntok)


def tune(threads: int) -> None:
    """Threads per CTA of the transfer kernel for the whole process (32 .. 256). With ``max_blocks`` = one CTA per SM and
    64 threads a transfer that runs beside a GEMM is spread evenly over the SMs instead of slowing a few of them."""
    _lib.call("slime_kv_tune", int(threads))


def kv_move(tok_k: int, tok_v: int, page_k: int, page_v: int, tok_off: torch.Tensor, blk: torch.Tensor,
            ntok: torch.Tensor | None, *, page_tokens: int, row_bytes: int, tok_rows: int, page_blocks: int,
            to_paged: bool = True, done_flag: int | None = None, done_value: int = 0, counter: torch.Tensor | None = None,
            max_blocks: int = 0, stream=None) -> None:
    """Launch one K+V page move (addresses are integers; the paged side may be a peer mapping)."""
    _lib.call("slime_kv_transfer", tok_k, tok_v, page_k, page_v, ptr(tok_off), ptr(blk), ptr(ntok), tok_off.numel(),
              page_tokens, row_bytes, tok_rows, page_blocks, int(to_paged), done_flag, done_value, ptr(counter),
              max_blocks, default_status().dev_ptr, stream_ptr(stream))


def kv_pack(tokens_kv: torch.Tensor, paged_kv: torch.Tensor, tok_off, blk, ntok=None) -> None:
    """token-major ``[2, tokens, row]`` -> paged ``[2, blocks, page_tokens, row]`` (local)."""
    _, rows, row = tokens_kv.shape
    _, blocks, page_tokens, _ = paged_kv.shape
    rb = row * tokens_kv.element_size()
    kv_move(tokens_kv[0].data_ptr(), tokens_kv[1].data_ptr(), paged_kv[0].data_ptr(), paged_kv[1].data_ptr(), tok_off, blk,
            ntok, page_tokens=page_tokens, row_bytes=rb, tok_rows=rows, page_blocks=blocks, to_paged=True)


def kv_unpack(paged_kv: torch.Tensor, tokens_kv: torch.Tensor, tok_off, blk, ntok=None) -> None:
    """paged -> token-major (local)."""
    _, rows, row = tokens_kv.shape
    _, blocks, page_tokens, _ = paged_kv.shape
    rb = row * tokens_kv.element_size()
    kv_move(tokens_kv[0].data_ptr(), tokens_kv[1].data_ptr(), paged_kv[0].data_ptr(), paged_kv[1].data_ptr(), tok_off, blk,
            ntok, page_tokens=page_tokens, row_bytes=rb, tok_rows=rows, page_blocks=blocks, to_paged=False)
