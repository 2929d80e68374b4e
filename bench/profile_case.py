#!/usr/bin/env python
"""Small, self-terminating cases for profiler captures (one or a few launches of one kernel).

    python bench/profile_case.py gemm        # 4096 x 4096 x 4096 bf16 GEMM, 3 launches
    python bench/profile_case.py gemm_pair   # the same product on CTA pairs (cta_group::2), 3 launches
    python bench/profile_case.py gemm_wide   # 8192^3 on CTA pairs with 256 x 512 tiles (operands larger than L2), 2 launches
    python bench/profile_case.py grouped_pair  # grouped SwiGLU gate/up + down GEMM on CTA pairs, 8 experts x 1024 rows, 2 launches each
    python bench/profile_case.py grouped_decode  # gate/up GEMM of a decode step on 8 ranks (32 experts x 32 rows): 128-row tiles, then 64-row tiles with five stages
    python bench/profile_case.py gemm_fp8    # the same shape in block-scaled fp8 (e4m3), 3 launches
    python bench/profile_case.py grouped     # grouped SwiGLU gate/up + down GEMM, 8 experts x 512 rows, 2 launches each
    python bench/profile_case.py grouped_stream  # the same GEMMs with 16 experts x 128 rows: weight streaming, HBM-bound
    python bench/profile_case.py moe_step    # one single-GPU MoE layer step (T=1024, 32 experts of the 7168/2048 shape)
    python bench/profile_case.py quant       # fp8 1x128 quantise + dequantise of 16384 x 7168
    python bench/profile_case.py copy        # 1024 x 64 KiB segment batch through the NVLink endpoint (local peer)
    python bench/profile_case.py kv          # paged KV pack + unpack, 4096 pages of 64 tokens x 512 B rows (K and V)
    python bench/profile_case.py allgather   # all-gather push of 1024 x 7168 bf16 to 4 emulated ranks on one GPU
    python bench/profile_case.py alltoall    # all-to-all of 4 x 512 x 7168 bf16 among 4 emulated ranks on one GPU
    python bench/profile_case.py ag_gemm_fused      # fused all-gather -> GEMM of rank 0 in a group of 4 emulated ranks (CTA pairs)
    python bench/profile_case.py ag_gemm_fp8_fused  # the same in block-scaled fp8
    python bench/profile_case.py moe_stream  # MoE step, streamed form: push + receive kernel and the gated GEMM (T=1024, 32 experts)

Each case holds well under 4 GB on the device and exits by itself in seconds.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def gemm_case():
    from dlslime_b200.ops import gemm

    a = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
    b = (torch.randn(4096, 4096, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm.gemm_bf16(a, b, out=out, pair=False)


def gemm_pair_case():
    from dlslime_b200.ops import gemm

    a = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
    b = (torch.randn(4096, 4096, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm.gemm_bf16_pair(a, b, out=out)


def gemm_wide_case():
    from dlslime_b200.ops import gemm

    a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    b = (torch.randn(8192, 8192, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm.gemm_bf16_pair(a, b, out=out, wide=True)


def grouped_pair_case():
    from dlslime_b200.ops import gemm

    g, rows, k, inter = 8, 1024, 7168, 2048
    offs = torch.arange(0, g + 1, dtype=torch.int32, device="cuda") * rows
    x = torch.randn(g * rows, k, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(g, k, inter, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(g * rows, inter, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(g * rows, k, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, pair=True)
        gemm.grouped_gemm_bf16(h, w2, offs, out=y, pair=True)


def grouped_decode_case():
    """Weight streaming with a few dozen rows per expert: the same launch with four 48 KB stages and with five 40 KB stages."""
    from dlslime_b200.ops import gemm

    g, rows, k, inter = 32, 32, 7168, 2048
    offs = torch.arange(0, g + 1, dtype=torch.int32, device="cuda") * rows
    x = torch.randn(g * rows, k, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(g * rows, inter, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU)
        gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU, tile_m=64)


def gemm_fp8_case():
    from dlslime_b200.ops import gemm, quant

    a = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
    b = (torch.randn(4096, 4096, device="cuda") * 0.02).to(torch.bfloat16)
    aq, sa = quant.fp8_quant_1x128(a)
    bq, sb = quant.fp8_quant_128x128(b)
    out = torch.empty(4096, 4096, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        gemm.gemm_fp8_blockscaled(aq, sa, bq, sb, out=out)


def grouped_case():
    from dlslime_b200.ops import gemm

    g, rows, k, inter = 8, 512, 7168, 2048
    offs = torch.arange(0, g + 1, dtype=torch.int32, device="cuda") * rows
    x = torch.randn(g * rows, k, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(g, k, inter, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(g * rows, inter, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(g * rows, k, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU)
        gemm.grouped_gemm_bf16(h, w2, offs, out=y)


def grouped_stream_case():
    """The weight-streaming regime of the expert GEMMs (few rows per expert, as on one GPU with 256 experts)."""
    from dlslime_b200.ops import gemm

    g, rows, k, inter = 16, 128, 7168, 2048
    offs = torch.arange(0, g + 1, dtype=torch.int32, device="cuda") * rows
    x = torch.randn(g * rows, k, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn(g, 2 * inter, k, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(g, k, inter, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(g * rows, inter, device="cuda", dtype=torch.bfloat16)
    y = torch.empty(g * rows, k, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        gemm.grouped_gemm_bf16(x, w13, offs, out=h, epilogue=gemm.EPI_SWIGLU)
        gemm.grouped_gemm_bf16(h, w2, offs, out=y)


def moe_case():
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig

    cfg = MoEConfig(num_experts=32, topk=8, hidden=7168, intermediate=2048)
    layer = ExpertParallelMoE(cfg, max_tokens=1024)
    x = torch.randn(1024, cfg.hidden, device="cuda").to(torch.bfloat16)
    lg = torch.randn(1024, cfg.num_experts, device="cuda")
    for _ in range(2):
        layer(x, lg)


def quant_case():
    from dlslime_b200.ops import quant

    x = torch.randn(16384, 7168, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        q, s = quant.fp8_quant_1x128(x)
        quant.fp8_dequant_1x128(q, s)


def copy_case():
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    n, seg = 1024, 64 << 10
    src = torch.randint(0, 255, (n * seg * 2,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(n * seg, dtype=torch.uint8, device="cuda")
    a, b = NVLinkEndpoint(), NVLinkEndpoint()
    a.register_memory_region(dst.data_ptr(), 0, dst.numel(), "dst")
    b.register_memory_region(src.data_ptr(), 0, src.numel(), "src")
    a.connect(b.endpoint_info())
    perm = torch.randperm(2 * n)[:n].tolist()
    for _ in range(2):
        a.read([("dst", "src", p * seg, i * seg, seg) for i, p in enumerate(perm)]).wait()
    a.close()
    b.close()


def kv_case():
    from dlslime_b200.ops import kv

    page, row, pages = 64, 256, 4096  # two KV heads of 128 per rank, as a TP4 shard of an 8-KV-head model
    tokens = page * pages
    src = torch.randn(2, tokens, row, device="cuda").to(torch.bfloat16)
    paged = torch.zeros(2, pages, page, row, device="cuda", dtype=torch.bfloat16)
    back = torch.empty_like(src)
    tok_off, blk, ntok = kv.build_page_tasks([tokens], page, torch.randperm(pages).tolist())
    for _ in range(2):
        kv.kv_pack(src, paged, tok_off, blk, ntok)
        kv.kv_unpack(paged, back, tok_off, blk, ntok)
    torch.cuda.synchronize()
    assert torch.equal(back, src)


def allgather_case():
    from dlslime_b200.ops.allgather import AllGatherLLBuffer

    world, bs, hidden = 4, 1024, 7168
    group = AllGatherLLBuffer.emulated_group(world, bs, hidden, torch.bfloat16)
    xs = [torch.randn(bs, hidden, device="cuda").to(torch.bfloat16) for _ in range(world)]
    for _ in range(2):
        hooks = [g.all_gather_ll_hook(x) for g, x in zip(group, xs)]
        outs = [h() for h in hooks]
    torch.cuda.synchronize()
    group[0].status.check()
    assert torch.equal(outs[0], torch.cat(xs, dim=0))


def alltoall_case():
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    world, bs, hidden = 4, 512, 7168
    group = AllToAllLLBuffer.emulated_group(world, bs, hidden, torch.bfloat16)
    xs = [torch.randn(world * bs, hidden, device="cuda").to(torch.bfloat16) for _ in range(world)]
    for _ in range(2):
        hooks = [g.all_to_all_ll_hook(x) for g, x in zip(group, xs)]
        outs = [h() for h in hooks]
    torch.cuda.synchronize()
    group[0].status.check()
    assert torch.equal(outs[1], torch.cat([x[bs:2 * bs] for x in xs], dim=0))


def ag_gemm_fused_case():
    """Rank 0's fused kernel in a group of four ranks that live on this one GPU: the other ranks push their shards with
    the push-only kernel first, so every arrival counter the fused kernel waits for is already complete, while its own
    push warps still copy rank 0's shard into all four regions beside the tensor-core tiles."""
    from dlslime_b200.ops.ag_gemm import AllGatherGemm

    world, rows, k, n = 4, 1024, 8192, 7168
    group = AllGatherGemm.emulated_group(world, rows, k)
    xs = [torch.randn(rows, k, device="cuda").to(torch.bfloat16) for _ in range(world)]
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(world * rows, n, device="cuda", dtype=torch.bfloat16)
    for step in (1, 2, 3):
        for g, x in zip(group[1:], xs[1:]):
            g.push(x, step)
        group[0]._call(3, xs[0], w, out, step)
    torch.cuda.synchronize()
    group[0].status.check()
    ref = torch.cat(xs, 0)[:256].float() @ w.float().t()
    assert ((out[:256].float() - ref).abs() <= ref.abs() * 2 ** -6 + ref.abs().mean() * 2 ** -6).all()


def ag_gemm_fp8_fused_case():
    from dlslime_b200.ops import quant
    from dlslime_b200.ops.ag_gemm import AllGatherGemmFp8

    world, rows, k, n = 4, 1024, 8192, 7168
    group = AllGatherGemmFp8.emulated_group(world, rows, k)
    xs = [quant.fp8_quant_1x128(torch.randn(rows, k, device="cuda").to(torch.bfloat16)) for _ in range(world)]
    wq, sb = quant.fp8_quant_128x128((torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16))
    out = torch.empty(world * rows, n, device="cuda", dtype=torch.bfloat16)
    for step in (1, 2, 3):
        for g, (xq, sx) in zip(group[1:], xs[1:]):
            g.push(xq, sx, step)
        group[0]._call(2, xs[0][0], xs[0][1], wq, sb, out, step)
    torch.cuda.synchronize()
    group[0].status.check()


def moe_stream_case():
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig

    cfg = MoEConfig(num_experts=32, topk=8, hidden=7168, intermediate=2048)
    layer = ExpertParallelMoE(cfg, max_tokens=1024, streamed=True)
    x = torch.randn(1024, cfg.hidden, device="cuda").to(torch.bfloat16)
    lg = torch.randn(1024, cfg.num_experts, device="cuda")
    for _ in range(3):
        layer(x, lg)
    torch.cuda.synchronize()
    layer.buf.status.check()


if __name__ == "__main__":
    {"ag_gemm_fused": ag_gemm_fused_case, "ag_gemm_fp8_fused": ag_gemm_fp8_fused_case, "moe_stream": moe_stream_case,
     "alltoall": alltoall_case, "kv": kv_case, "allgather": allgather_case, "gemm": gemm_case, "gemm_pair": gemm_pair_case, "gemm_wide": gemm_wide_case,
     "grouped_pair": grouped_pair_case, "grouped_decode": grouped_decode_case, "gemm_fp8": gemm_fp8_case, "grouped": grouped_case, "grouped_stream": grouped_stream_case, "moe_step": moe_case, "quant": quant_case, "copy": copy_case}[sys.argv[1]]()
    torch.cuda.synchronize()
    print("done", sys.argv[1])
