#!/usr/bin/env python
"""Multi-GPU benchmarks of the communication kernels against library baselines (one rank per GPU).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 --master-port 29650 bench/comm_bench.py <case>

Cases (shapes from the benchmark definition of this project):
  p2p        NVLink endpoint: contiguous read and write 8 B ... 1 GiB between rank pairs (r, r^1), and a batched
             scatter of 4096 x 64 KiB segments at permuted offsets; baseline = one cudaMemcpyAsync per segment
             (what the reference's NVLinkEndpoint.read does per assignment).
  p2p_scatter  only the batched scatter of the p2p case.
  allgather  low-latency all-gather of [T, 7168] bf16, T in {1, 16, 128, 1024}; baseline = NCCL all_gather_into_tensor.
  alltoall   low-latency all-to-all of [world * T, 7168] bf16, T in {1, 16, 128, 512}; baseline = NCCL all_to_all_single.
  ag_gemm_fp8  the same shape in e4m3 with 1x128 / 128x128 block scales (fp8 payload + scales cross NVLink)
  ag_gemm    per-rank [1024, 8192] bf16 gathered and multiplied by W[28672 / world, 8192]; fused kernel vs
             NCCL all-gather + torch.matmul (cuBLAS).
  p2p_pairs  contiguous read and write 8 B ... 1 GiB over EVERY ordered pair of GPUs (min / median / max per size).
  agg        the reference's aggregate SPMD shape: half the ranks initiate, batch x concurrency, summed MB/s.
  kv_cache   DLSlimeCache put / get of the KV pages of the kv case with the cache's slabs in GPU memory.
  kv         TP(world/2) -> TP(world/2) transfer of a 32-layer, 64-token-page KV cache for 16 prompts of
             512..8192 tokens, layer by layer, overlapped with a bf16 GEMM chain; baseline = one copy per page.

Every number is timed with CUDA events on the launching stream after warm-up, taken as the maximum over ranks,
and printed by rank 0 as one JSON line per measurement.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def max_ms(ms, world):
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed(fn, iters, warmup=3, sync=None):
    for _ in range(warmup):
        fn()
    if sync:
        sync()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def emit(rank, **kw):
    if rank == 0:
        print(json.dumps(kw), flush=True)


# ------------------------------------------------------------------------------------------ all-to-all
def case_alltoall(rank, world):
    """Low-latency all-to-all of [world * T, 7168] bf16 (T rows to every rank) against NCCL all_to_all_single."""
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    hidden = 7168
    a2a = AllToAllLLBuffer(512, hidden, torch.bfloat16)
    for T in (1, 16, 128, 512):
        x = torch.randn(world * T, hidden, device="cuda").to(torch.bfloat16)
        ref = torch.empty_like(x)
        ms = max_ms(timed(lambda: a2a.all_to_all_ll(x), 200, sync=dist.barrier), world)
        dist.barrier()
        base = max_ms(timed(lambda: dist.all_to_all_single(ref, x), 200, sync=dist.barrier), world)
        a2a.status.check()
        nbytes = T * hidden * 2 * (world - 1)
        emit(rank, case="ll_alltoall", T=T, world=world, us=round(ms * 1e3, 2), nccl_us=round(base * 1e3, 2), speedup=round(base / ms, 2),
             send_gbs_per_rank=round(nbytes / ms / 1e6, 1), frac_of_nvlink=round(nbytes / ms / 1e6 / NVLINK_GBS, 3))


# ------------------------------------------------------------------------------------------ p2p
def case_p2p(rank, world, contiguous=True):
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    peer = rank ^ 1
    big = 1 << 30
    region = 4 << 30
    local = torch.empty(region, dtype=torch.uint8, device="cuda")
    # every byte of the region is written once before anything is timed: a transfer engine moves data that somebody produced
    for o in range(0, region, 1 << 28):
        local[o:o + (1 << 28)].random_(0, 255)
    torch.cuda.synchronize()
    ep = NVLinkEndpoint()
    ep.register_memory_region(local.data_ptr(), 0, region, "buf")
    infos = [None] * world
    dist.all_gather_object(infos, ep.endpoint_info())
    ep.connect(infos[peer])
    # baseline path: peer pointer through torch's own peer mapping is not available across processes, so the
    # per-segment cudaMemcpyAsync baseline reuses the endpoint's mapped peer address
    import ctypes

    from dlslime_b200 import _lib

    lib = _lib.load()
    lib.slime_nvlink_ep_remote_addr.restype = ctypes.c_ulonglong
    peer_addr = lib.slime_nvlink_ep_remote_addr(ep._h, ep.get_remote_mr_handle("buf"))
    memcpy = lib.slime_memcpy_async  # plain cudaMemcpyAsync, the per-segment baseline
    rbuf, lbuf = ep.get_remote_mr_handle("buf"), ep.get_mr_handle("buf")
    dist.barrier()
    active = rank < peer  # one direction per pair at a time
    sizes = [8 << i for i in range(0, 28)] if contiguous else []  # 8 B ... 1 GiB
    for op in ("read", "write"):
        for n in sizes:
            iters = 200 if n <= (1 << 20) else 20 if n <= (1 << 26) else 5
            if active:
                fn = (lambda: ep.read([(lbuf, rbuf, 0, 0, n)], want_future=False)) if op == "read" else (lambda: ep.write([(lbuf, rbuf, 0, 0, n)], want_future=False))
                ms = timed(fn, iters)
                src, dst = (peer_addr, local.data_ptr()) if op == "read" else (local.data_ptr(), peer_addr)
                base = timed(lambda: memcpy(dst, src, n, torch.cuda.current_stream().cuda_stream), iters)
            else:
                ms = base = 0.0
            dist.barrier()
            ms, base = max_ms(ms, world), max_ms(base, world)
            emit(rank, case="p2p_contiguous", op=op, bytes=n, us=round(ms * 1e3, 2), gbs=round(n / ms / 1e6, 2),
                 baseline_memcpy_us=round(base * 1e3, 2), baseline_gbs=round(n / base / 1e6, 2),
                 frac_of_nvlink=round(n / ms / 1e6 / NVLINK_GBS, 3), world=world)
    # batched scatter: 4096 x 64 KiB at permuted offsets of the 4 GiB remote region
    seg, nseg = 64 << 10, 4096
    g = torch.Generator().manual_seed(0)
    perm = torch.randperm(region // seg, generator=g)[:nseg].tolist()
    assign = [(lbuf, rbuf, p * seg, i * seg, seg) for i, p in enumerate(perm)]
    import numpy as np

    arr = np.ascontiguousarray(np.asarray(assign, dtype=np.uint64))
    for op in ("read", "write"):
        if active:
            fn = (lambda: ep._transfer(arr, op == "write", None, want_future=False))
            ms = timed(fn, 10, warmup=5)

            def loop():
                s = torch.cuda.current_stream().cuda_stream
                for i, p in enumerate(perm):
                    if op == "read":
                        memcpy(local.data_ptr() + i * seg, peer_addr + p * seg, seg, s)
                    else:
                        memcpy(peer_addr + p * seg, local.data_ptr() + i * seg, seg, s)

            base = timed(loop, 3, warmup=1)
        else:
            ms = base = 0.0
        dist.barrier()
        ms, base = max_ms(ms, world), max_ms(base, world)
        tot = seg * nseg
        emit(rank, case="p2p_scatter_4096x64KiB", op=op, bytes=tot, us=round(ms * 1e3, 1), gbs=round(tot / ms / 1e6, 1),
             baseline_memcpy_loop_us=round(base * 1e3, 1), baseline_gbs=round(tot / base / 1e6, 1), speedup=round(base / ms, 2),
             frac_of_nvlink=round(tot / ms / 1e6 / NVLINK_GBS, 3), world=world)
    if os.environ.get("SLIME_P2P_SWEEP", "0") == "1":
        # what limits the scattered read: work unit (CTAs per 64 KiB piece), grid size, copy mechanism
        from dlslime_b200.ops import nvlink as nv

        for op in ("read", "write"):
            for bulk in (1, 0):
                for unit_kb in (16, 32, 64):
                    for blocks in (0, 74, 148, 296, 592):
                        nv.tune(unit_kb, bulk)
                        ms = timed(lambda: ep._transfer(arr, op == "write", None, want_future=False, max_blocks=blocks), 10) if active else 0.0
                        dist.barrier()
                        ms = max_ms(ms, world)
                        emit(rank, case="p2p_scatter_sweep", op=op, bulk=bulk, unit_kb=unit_kb, max_blocks=blocks,
                             us=round(ms * 1e3, 1), gbs=round(seg * nseg / ms / 1e6, 1))
        nv.tune(64, 1)
    dist.barrier()
    ep.close()


# ------------------------------------------------------------------------------------------ p2p, every pair
def case_p2p_pairs(rank, world):
    """Contiguous read and write, 8 B ... 1 GiB, over EVERY ordered pair of GPUs. Round k pairs rank r with r ^ k
    (disjoint pairs, so the rounds of one k run at the same time without sharing a link); in each round first the
    lower rank of a pair initiates, then the higher. Per size and operation the minimum, median and maximum over all
    ordered pairs are printed, with the slowest pair."""
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    region = 1 << 30
    local = torch.empty(region, dtype=torch.uint8, device="cuda")
    for o in range(0, region, 1 << 28):
        local[o:o + (1 << 28)].random_(0, 255)
    torch.cuda.synchronize()
    eps = {}
    infos_all = [None] * world
    mine = {}
    for peer in range(world):
        if peer != rank:
            ep = NVLinkEndpoint()
            ep.register_memory_region(local.data_ptr(), 0, region, "buf")
            eps[peer] = ep
            mine[peer] = ep.endpoint_info()
    dist.all_gather_object(infos_all, mine)
    for peer, ep in eps.items():
        ep.connect(infos_all[peer][rank])
    dist.barrier()
    sizes = [8 << i for i in range(0, 28)]
    results = {}  # (op, size) -> list of (gbs, us, src, dst) gathered on rank 0
    for k in range(1, 1 << (world - 1).bit_length()):
        peer = rank ^ k
        if peer >= world:
            peer = None
        for lower_first in (True, False):
            active = peer is not None and ((rank < peer) == lower_first)
            row = []
            for op in ("read", "write"):
                for n in sizes:
                    iters = 100 if n <= (1 << 20) else 10 if n <= (1 << 26) else 3
                    if active:
                        ep = eps[peer]
                        lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
                        fn = (lambda: ep.read([(lh, rh, 0, 0, n)], want_future=False)) if op == "read" else (lambda: ep.write([(lh, rh, 0, 0, n)], want_future=False))
                        ms = timed(fn, iters, warmup=2)
                        row.append((op, n, ms))
                    dist.barrier()
            gathered = [None] * world
            dist.all_gather_object(gathered, (rank, peer, row) if active else None)
            if rank == 0:
                for g in gathered:
                    if g:
                        src, dst, rows = g
                        for op, n, ms in rows:
                            results.setdefault((op, n), []).append((n / ms / 1e6, ms * 1e3, src, dst))
    if rank == 0:
        for op in ("read", "write"):
            for n in sizes:
                v = sorted(results[(op, n)])
                med = v[len(v) // 2]
                emit(0, case="p2p_every_pair", op=op, bytes=n, pairs=len(v), us_median=round(med[1], 2), gbs_min=round(v[0][0], 2),
                     gbs_median=round(med[0], 2), gbs_max=round(v[-1][0], 2), slowest_pair=[v[0][2], v[0][3]], world=world)
    dist.barrier()
    for ep in eps.values():
        ep.close()


# ------------------------------------------------------------------------------------------ aggregate transfer, SPMD
def case_agg(rank, world):
    """The reference's aggregate transfer benchmark shape (bench/python/agg_transfer_bench_spmd.py:76-84,292-317,475-497 in
    the reference): the lower half of the ranks initiate, rank r reading from rank r + world/2; message sizes 2 << n
    fp32 elements for n in [8, 19]; every iteration posts `concurrency` operations of `batch` identical assignments
    each and waits for all of them; 10 warm-up and 100 timed iterations between CUDA events; the bandwidth is summed
    over the initiators. Baseline: the same with one cudaMemcpyAsync per assignment (the reference endpoint's method)."""
    import ctypes

    from dlslime_b200 import _lib
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    half = world // 2
    initiator = rank < half
    peer = rank + half if initiator else rank - half
    max_bytes = (2 << 19) * 4
    region = max_bytes * 64
    local = torch.empty(region, dtype=torch.uint8, device="cuda")
    local.random_(0, 255)
    ep = NVLinkEndpoint()
    ep.register_memory_region(local.data_ptr(), 0, region, "buf")
    infos = [None] * world
    dist.all_gather_object(infos, ep.endpoint_info())
    ep.connect(infos[peer])
    lib = _lib.load()
    lib.slime_nvlink_ep_remote_addr.restype = ctypes.c_ulonglong
    peer_addr = lib.slime_nvlink_ep_remote_addr(ep._h, ep.get_remote_mr_handle("buf"))
    memcpy = lib.slime_memcpy_async
    lh, rh = ep.get_mr_handle("buf"), ep.get_remote_mr_handle("buf")
    dist.barrier()
    for batch, conc in ((1, 1), (64, 1), (64, 8)):
        for n in range(8, 20):
            nbytes = (2 << n) * 4
            assign = [(lh, rh, (i % 64) * nbytes, (i % 64) * nbytes, nbytes) for i in range(batch)]

            def ours():
                futs = [ep.read(assign) for _ in range(conc)]
                for f in futs:
                    f.wait(30.0)

            def per_assignment():
                s = torch.cuda.current_stream().cuda_stream
                for _ in range(conc):
                    for (_l, _r, ro, lo, nb) in assign:
                        memcpy(local.data_ptr() + lo, peer_addr + ro, nb, s)
                torch.cuda.current_stream().synchronize()

            ms = timed(ours, 100, warmup=10) if initiator else 0.0
            dist.barrier()
            base = timed(per_assignment, 20, warmup=3) if initiator else 0.0
            dist.barrier()
            tot = nbytes * batch * conc
            t = torch.tensor([tot / ms / 1e3 if initiator else 0.0, tot / base / 1e3 if initiator else 0.0, ms, base], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)  # sums the initiators' MB/s
            emit(rank, case="agg_transfer_spmd", world=world, initiators=half, batch=batch, concurrency=conc, bytes=nbytes,
                 avg_latency_ms=round(float(t[2]) / half, 4), agg_mbs=round(float(t[0]), 1), per_assignment_memcpy_agg_mbs=round(float(t[1]), 1),
                 speedup=round(float(t[0]) / max(float(t[1]), 1e-9), 2))
    dist.barrier()
    ep.close()


# ------------------------------------------------------------------------------------------ all-gather
def case_allgather(rank, world):
    from dlslime_b200.ops.allgather import AllGatherLLBuffer

    hidden = 7168
    # SLIME_AG_MULTICAST = always | never | auto: multimem stores through the switch, plain peer stores, or by size
    ag = AllGatherLLBuffer(1024, hidden, torch.bfloat16, multicast=None)
    emit(rank, case="ll_allgather_setup", multicast_heap=bool(ag.use_multicast), policy=os.environ.get("SLIME_AG_MULTICAST", "auto"))
    for T in (1, 16, 128, 1024):
        x = torch.randn(T, hidden, device="cuda").to(torch.bfloat16)
        ref = torch.empty(world * T, hidden, device="cuda", dtype=torch.bfloat16)
        ms = max_ms(timed(lambda: ag.all_gather_ll(x), 200, sync=dist.barrier), world)
        dist.barrier()
        base = max_ms(timed(lambda: dist.all_gather_into_tensor(ref, x), 200, sync=dist.barrier), world)
        ag.status.check()
        # device-only latency: 20 calls captured in a CUDA graph each, so host launch cost drops out on both sides
        def graph_us(fn):
            g = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                fn()
                fn()
            torch.cuda.current_stream().wait_stream(s)
            dist.barrier()
            with torch.cuda.graph(g):
                for _ in range(20):
                    fn()
            return timed(g.replay, 10, sync=dist.barrier) / 20

        try:
            g_ms = max_ms(graph_us(lambda: ag.all_gather_ll(x)), world)
            g_base = max_ms(graph_us(lambda: dist.all_gather_into_tensor(ref, x)), world)
        except Exception as e:  # graph capture of either side not possible here
            g_ms = g_base = float("nan")
            if rank == 0:
                print("graph timing skipped:", e, flush=True)
        nbytes = T * hidden * 2 * (world - 1)
        emit(rank, case="ll_allgather", multicast=bool(ag._through_multicast(T * hidden * 2)), T=T, world=world, us=round(ms * 1e3, 2), nccl_us=round(base * 1e3, 2), speedup=round(base / ms, 2),
             graph_us=round(g_ms * 1e3, 2), nccl_graph_us=round(g_base * 1e3, 2),
             recv_gbs_per_rank=round(nbytes / ms / 1e6, 1), frac_of_nvlink=round(nbytes / ms / 1e6 / NVLINK_GBS, 3))


# ------------------------------------------------------------------------------------------ ag + gemm
def case_ag_gemm(rank, world):
    from dlslime_b200.ops.ag_gemm import AllGatherGemm

    _, tf, tag = peaks()
    rows, k, n = 1024, 8192, 28672 // world
    ag = AllGatherGemm(rows, k)
    x = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(world * rows, n, device="cuda", dtype=torch.bfloat16)
    full = torch.empty(world * rows, k, device="cuda", dtype=torch.bfloat16)

    def fused():
        ag.forward(x, w, out)
        dist.barrier()  # the gathered matrix may be overwritten only after every rank consumed it

    def baseline():
        dist.all_gather_into_tensor(full, x)
        torch.matmul(full, w.t(), out=out)
        dist.barrier()

    def barrier_only():
        dist.barrier()

    # the two halves on their own, as separate kernels: the push of this rank's shard to every rank, and the
    # gated GEMM over the gathered matrix once everything has arrived (its counters are already satisfied)
    def push_only():
        ag.step += 1
        ag.push(x, ag.step, push_blocks=148)
        dist.barrier()

    def gemm_only():
        ag.gemm(w, out, ag.step)

    def local_gemm():
        gemm.gemm_bf16(full, w, out=out)

    from dlslime_b200.ops import gemm

    b = timed(barrier_only, 50, sync=dist.barrier)
    ms = max_ms(timed(fused, 50, sync=dist.barrier) - b, world)
    base = max_ms(timed(baseline, 50, sync=dist.barrier) - b, world)
    push_ms = max_ms(timed(push_only, 20, sync=dist.barrier) - b, world)
    gemm_ms = max_ms(timed(gemm_only, 20, sync=dist.barrier), world)
    plain_ms = max_ms(timed(local_gemm, 20, sync=dist.barrier), world)
    ag.status.check()
    flops = 2.0 * world * rows * k * n
    gathered = (world - 1) * rows * k * 2
    roof_ms = max(flops / (tf * 1e9), gathered / (NVLINK_GBS * 1e6))
    emit(rank, case="ag_gemm_bf16", world=world, M=world * rows, N=n, K=k, us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 1),
         nccl_cublas_us=round(base * 1e3, 1), speedup=round(base / ms, 2), roofline_us=round(roof_ms * 1e3, 1),
         frac_of_roofline=round(roof_ms / ms, 3), peak=tag, push_kernel_alone_us=round(push_ms * 1e3, 1),
         gated_gemm_alone_us=round(gemm_ms * 1e3, 1), plain_gemm_same_shape_us=round(plain_ms * 1e3, 1))


def case_ag_gemm_fp8(rank, world):
    """The same shape in e4m3 with 1x128 / 128x128 block scales: quantise + fused kernel vs NCCL all-gather of the
    fp8 payload and scales + the block-scaled GEMM alone, and vs the bf16 fused kernel."""
    from dlslime_b200.ops import gemm, quant
    from dlslime_b200.ops.ag_gemm import AllGatherGemm, AllGatherGemmFp8

    _, tf, tag = peaks()
    rows, k, n = 1024, 8192, 28672 // world
    ag = AllGatherGemmFp8(rows, k)
    ag16 = AllGatherGemm(rows, k)
    x = torch.randn(rows, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    wq, sb = quant.fp8_quant_128x128(w)
    out = torch.empty(world * rows, n, device="cuda", dtype=torch.bfloat16)
    fq = torch.empty(world * rows, k, device="cuda", dtype=torch.uint8)
    fs = torch.empty(world * rows, k // 128, device="cuda", dtype=torch.float32)

    def fused():
        ag.forward(x, wq, sb, out)
        dist.barrier()

    def fused_bf16():
        ag16.forward(x, w, out)
        dist.barrier()

    def baseline():
        xq, sx = quant.fp8_quant_1x128(x)
        dist.all_gather_into_tensor(fq, xq.view(torch.uint8))
        dist.all_gather_into_tensor(fs, sx)
        gemm.gemm_fp8_blockscaled(fq.view(torch.float8_e4m3fn), fs, wq, sb, out=out)
        dist.barrier()

    def gemm_alone():
        gemm.gemm_fp8_blockscaled(fq.view(torch.float8_e4m3fn), fs, wq, sb, out=out)

    b = timed(lambda: dist.barrier(), 50, sync=dist.barrier)
    ms = max_ms(timed(fused, 50, sync=dist.barrier) - b, world)
    ms16 = max_ms(timed(fused_bf16, 50, sync=dist.barrier) - b, world)
    base = max_ms(timed(baseline, 50, sync=dist.barrier) - b, world)
    alone = max_ms(timed(gemm_alone, 20, sync=dist.barrier), world)
    ag.status.check()
    flops = 2.0 * world * rows * k * n
    emit(rank, case="ag_gemm_fp8_blockscaled", world=world, M=world * rows, N=n, K=k, us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 1),
         includes="1x128 quantisation of the local shard", bf16_fused_us=round(ms16 * 1e3, 1),
         nccl_plus_fp8_gemm_us=round(base * 1e3, 1), speedup_vs_nccl=round(base / ms, 2), fp8_gemm_alone_us=round(alone * 1e3, 1),
         nvlink_bytes_in_per_rank=(world - 1) * rows * (k + k // 128 * 4))


# ------------------------------------------------------------------------------------------ kv
def case_kv(rank, world):
    from dlslime_b200.models.pd_kv import KVShape, PagedKVCache, PrefillSender, wait_layers
    from dlslime_b200.ops import gemm
    from dlslime_b200.parallel.symm import SymmetricHeap

    half = world // 2
    shape = KVShape()  # 32 layers, 2 local KV heads, head_dim 128, 64-token pages
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(512, 8193, (16,), generator=g).tolist()
    pages = sum((n + 63) // 64 for n in lens)
    tokens = sum(lens)
    blocks = pages + 64
    heap = SymmetricHeap(PagedKVCache.bytes_needed(shape, blocks))
    is_prefill = rank < half
    cache = PagedKVCache(shape, blocks, heap, owner_rank=rank + half if is_prefill else rank)
    dst_blocks = torch.randperm(blocks, generator=torch.Generator().manual_seed(11 + rank % half))[:pages].tolist()
    total_bytes = 2 * shape.layers * tokens * shape.row_bytes
    res = {}
    if is_prefill:
        # SLIME_KV_COMM = "blocks,threads" of the transfer kernel (default 148,64: one thin CTA per SM)
        cb, ct = (int(v) for v in os.environ.get("SLIME_KV_COMM", "148,64").split(","))
        sender = PrefillSender(shape, cache, max_tokens=tokens, comm_blocks=cb, comm_threads=ct)
        sender.kv_stage.normal_()
        d = 4096
        hidden = torch.randn(tokens, d, device="cuda").to(torch.bfloat16)
        weights = [(torch.randn(d, d, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(2)]
        tmp = torch.empty_like(hidden)

        def transfer_only():
            sender.plan(lens, dst_blocks)
            for layer in range(shape.layers):
                sender.send_layer(layer)

        def compute_only():
            a, b = hidden, tmp
            for layer in range(shape.layers):
                gemm.gemm_bf16(a, weights[layer % 2], out=b)
                a, b = b, a

        def overlapped():
            sender.plan(lens, dst_blocks)
            sender.run_prefill_with_transfer(hidden, weights, overlap=True)

        from dlslime_b200 import _lib

        memcpy = _lib.load().slime_memcpy_async
        tok_off, blk, ntok = sender.plan(lens, dst_blocks)
        to, bl, nt = tok_off.tolist(), blk.tolist(), ntok.tolist()

        def per_page_memcpy():
            s = torch.cuda.current_stream().cuda_stream
            for layer in range(shape.layers):
                for plane in range(2):
                    src0 = sender.kv_stage[layer, plane].data_ptr()
                    dst0 = cache.plane_addr(layer, plane)
                    for t, b, n in zip(to, bl, nt):
                        memcpy(dst0 + b * shape.page_bytes, src0 + t * shape.row_bytes, n * shape.row_bytes, s)

        res["transfer"] = timed(transfer_only, 5)
        # the chain is ~65 ms and power-capped, its run-to-run spread (~1 ms) is as large as the effect looked for:
        # alternate the two forms and take medians
        cs, ov = [], []
        for _ in range(7):
            cs.append(timed(compute_only, 1, warmup=1 if not cs else 0))
            ov.append(timed(overlapped, 1, warmup=1 if not ov else 0))
        res["compute"] = sorted(cs)[len(cs) // 2]
        res["overlap"] = sorted(ov)[len(ov) // 2]
        res["memcpy"] = timed(per_page_memcpy, 2, warmup=1)
    dist.barrier()
    vals = {k: max_ms(res.get(k, 0.0), world) for k in ("transfer", "compute", "overlap", "memcpy")}
    eff = (vals["transfer"] + vals["compute"] - vals["overlap"]) / min(vals["transfer"], vals["compute"]) if min(vals["transfer"], vals["compute"]) > 0 else 0
    emit(rank, case="pd_kv_transfer", world=world, prompts=16, tokens=tokens, pages=pages, bytes_per_rank=total_bytes,
         transfer_ms=round(vals["transfer"], 3), gbs_per_rank=round(total_bytes / vals["transfer"] / 1e6, 1),
         frac_of_nvlink=round(total_bytes / vals["transfer"] / 1e6 / NVLINK_GBS, 3),
         per_page_memcpy_ms=round(vals["memcpy"], 3), memcpy_gbs=round(total_bytes / vals["memcpy"] / 1e6, 1), speedup=round(vals["memcpy"] / vals["transfer"], 2),
         prefill_gemm_chain_ms=round(vals["compute"], 3), overlapped_ms=round(vals["overlap"], 3), overlap_efficiency=round(eff, 3),
         exposed_ms=round(vals["overlap"] - vals["compute"], 3), comm_grid=os.environ.get("SLIME_KV_COMM", "148,64"))
    if not is_prefill:
        assert wait_layers(cache, 1, timeout_s=30.0)
    dist.barrier()


def case_kv_cache(rank, world):
    """DLSlimeCache put / get of the same KV pages with the cache's slabs on a GPU: rank world/2 runs the cache service
    (directory + 3 GiB of slabs in its GPU's memory, reached over NVLink through a PeerAgent), rank 0 stores the K and V
    rows of all 16 prompts and 32 layers (one extent per layer, plane and prompt: 1024 extents, 2 GB) with
    ``CacheClient.put`` and reads them back with ``get``; both directions are checked byte for byte."""
    import time

    from dlslime_b200.cache import CacheClient
    from dlslime_b200.cache.service import CacheHttpServer, CacheService
    from dlslime_b200.models.pd_kv import KVShape
    from dlslime_b200.nanoctrl import start_local_nanoctrl
    from dlslime_b200.peer_agent import PeerAgent

    half = world // 2
    shape = KVShape()
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(512, 8193, (16,), generator=g).tolist()
    tokens = sum(lens)
    ctrl = start_local_nanoctrl() if rank == 0 else None
    urls = [None]
    if rank == 0:
        urls = [ctrl.url]
    dist.broadcast_object_list(urls, src=0)
    url = urls[0]
    srv = agent = None
    res = {}
    dev = f"cuda:{torch.cuda.current_device()}"
    if rank == half:
        agent = PeerAgent(url, alias="kv-cache", device=dev, link_type="nvlink")
        service = CacheService(agent, slab_size=1 << 20, memory_size=3 << 30, device=dev)
        srv = CacheHttpServer(service, host="127.0.0.1", port=0)
        srv.start()
        cache_url = [f"http://127.0.0.1:{srv.port}"]
    else:
        cache_url = [None]
    dist.broadcast_object_list(cache_url, src=half)
    if rank == 0:
        agent = PeerAgent(url, alias="prefill-0", device=dev, link_type="nvlink")
        stage = torch.empty((shape.layers, 2, tokens, shape.row), dtype=shape.dtype, device="cuda").normal_()
        back = torch.zeros_like(stage)
        nbytes = stage.numel() * 2
        agent.register_memory_region("kv", stage.data_ptr(), 0, nbytes)
        agent.register_memory_region("kv_back", back.data_ptr(), 0, nbytes)
        client = CacheClient(cache_url[0], peer_agent=agent, timeout=60.0)
        client.connect_to_server(link_type="nvlink")
        extents, t = [], 0
        for layer in range(shape.layers):
            for plane in range(2):
                t = 0
                for n in lens:
                    extents.append((((layer * 2 + plane) * tokens + t) * shape.row_bytes, n * shape.row_bytes))
                    t += n
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        manifest = client.put("kv", extents, timeout=120.0)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        client.get("kv_back", agent.alias, manifest["version"], timeout=120.0)
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        ok = bool(torch.equal(stage, back))
        res = {"put_ms": (t1 - t0) * 1e3, "get_ms": (t2 - t1) * 1e3, "bytes": nbytes, "extents": len(extents), "ok": ok}
        client.delete(agent.alias, manifest["version"])
    dist.barrier()
    out = [res]
    dist.broadcast_object_list(out, src=0)
    r = out[0]
    emit(rank, case="kv_cache_put_get_gpu_slabs", world=world, bytes=r["bytes"], extents=r["extents"], slab_bytes=1 << 20,
         put_ms=round(r["put_ms"], 2), put_gbs=round(r["bytes"] / r["put_ms"] / 1e6, 1), get_ms=round(r["get_ms"], 2),
         get_gbs=round(r["bytes"] / r["get_ms"] / 1e6, 1), bytes_equal=r["ok"],
         includes="the HTTP round trips to the directory (store / query) and the endpoint transfer of every slab piece")
    dist.barrier()
    if agent is not None:
        agent.shutdown()
    if srv is not None:
        srv.stop()
    dist.barrier()
    if ctrl is not None:
        ctrl.stop()


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29650")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), rank=rank, world_size=world)
    for case in sys.argv[1:]:
        {"p2p": case_p2p, "p2p_scatter": lambda r, w: case_p2p(r, w, contiguous=False), "allgather": case_allgather, "alltoall": case_alltoall, "ag_gemm": case_ag_gemm, "ag_gemm_fp8": case_ag_gemm_fp8, "kv": case_kv,
         "p2p_pairs": case_p2p_pairs, "agg": case_agg, "kv_cache": case_kv_cache}[case](rank, world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
