"""Multi-GPU checks, one process per GPU (launched by test_gpu_multi.py through torchrun).

Every check compares against a PyTorch / NCCL restatement of the same operation.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def check_endpoint(rank, world):
    from dlslime_b200.ops.nvlink import NVLinkEndpoint

    peer = rank ^ 1
    if peer >= world:
        return
    n = 8 << 20
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    buf = torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda", generator=gen)
    orig = buf.clone()
    ep = NVLinkEndpoint()
    ep.register_memory_region(buf.data_ptr(), 0, n, "buffer")
    infos = [None] * world
    dist.all_gather_object(infos, ep.endpoint_info())
    ep.connect(infos[peer])
    peer_gen = torch.Generator(device="cuda").manual_seed(100 + peer)
    peer_orig = torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda", generator=peer_gen)
    dist.barrier()
    half = n // 2
    if rank < peer:
        # read: pull scattered pieces of the peer's upper half into my lower half (odd sizes and offsets included)
        segs = [("buffer", "buffer", half + 1000 * i + (i % 3), 5000 * i + (i % 5), 777 + 16 * i) for i in range(200)]
        segs.append(("buffer", "buffer", half + (1 << 20), 1 << 20, 1 << 20))
        fut = ep.read(segs)
        assert fut.wait() == 0
        expect = orig.clone()
        for _, _, roff, loff, ln in segs:
            expect[loff:loff + ln] = peer_orig[roff:roff + ln]
        torch.cuda.synchronize()
        assert torch.equal(buf, expect), "endpoint read mismatch"
        # aligned batch (the bulk-copy-engine path): 40 scattered 64 KiB pieces, one 200 KiB piece, one 48-byte piece
        segs = [("buffer", "buffer", half + (1 << 20) + 65536 * ((7 * i) % 40), (2 << 20) + 65536 * i, 65536) for i in range(20)]
        segs += [("buffer", "buffer", half + 4096, 4096, 200 << 10), ("buffer", "buffer", half + 16, 1 << 19, 48)]
        assert ep.read(segs).wait() == 0
        for _, _, roff, loff, ln in segs:
            expect[loff:loff + ln] = peer_orig[roff:roff + ln]
        torch.cuda.synchronize()
        assert torch.equal(buf, expect), "endpoint bulk read mismatch"
        # one contiguous piece at odd offsets (the copy-engine route), by name and by handle
        one = ("buffer", "buffer", half + 12345, (3 << 20) + 7, 1_000_001)
        assert ep.read([one]).wait() == 0
        lh, rh = ep.get_mr_handle("buffer"), ep.get_remote_mr_handle("buffer")
        two = (lh, rh, half + 77, (3 << 20) - 4099, 4096)
        assert ep.read([two]).wait() == 0
        for _, _, roff, loff, ln in (one, two):
            expect[loff:loff + ln] = peer_orig[roff:roff + ln]
        torch.cuda.synchronize()
        assert torch.equal(buf, expect), "endpoint single-piece read mismatch"
    dist.barrier()
    if rank < peer:
        # write with immediate data: push my lower half into the peer's lower half, then notify
        lh, rh = ep.get_mr_handle("buffer"), ep.get_remote_mr_handle("buffer")
        fut = ep.write_with_imm([(lh, rh, 4096, 4096, half - 8192)], imm_data=0xBEEF)
        assert fut.wait() == 0
    else:
        status, imm = ep.imm_recv()
        assert status == 0 and imm == 0xBEEF, (status, imm)
        torch.cuda.synchronize()
        # what the peer wrote is ITS buffer after its own reads; recompute that
        psegs = [(half + 1000 * i + (i % 3), 5000 * i + (i % 5), 777 + 16 * i) for i in range(200)]
        psegs.append((half + (1 << 20), 1 << 20, 1 << 20))
        psegs += [(half + (1 << 20) + 65536 * ((7 * i) % 40), (2 << 20) + 65536 * i, 65536) for i in range(20)]
        psegs += [(half + 4096, 4096, 200 << 10), (half + 16, 1 << 19, 48)]
        psegs += [(half + 12345, (3 << 20) + 7, 1_000_001), (half + 77, (3 << 20) - 4099, 4096)]
        pbuf = peer_orig.clone()
        for roff, loff, ln in psegs:
            pbuf[loff:loff + ln] = orig[roff:roff + ln]
        assert torch.equal(buf[4096:half - 4096], pbuf[4096:half - 4096]), "endpoint write mismatch"
        assert torch.equal(buf[:4096], orig[:4096]) and torch.equal(buf[half:], orig[half:])
    dist.barrier()
    ep.close()


def check_allgather(rank, world):
    from dlslime_b200.ops.allgather import AllGatherLLBuffer

    hidden = 7168
    ag = AllGatherLLBuffer(1024, hidden, torch.bfloat16)
    for step, bs in enumerate([1, 16, 128, 1024, 16, 1]):
        x = torch.randn((bs, hidden), device="cuda").to(torch.bfloat16) + rank
        ref = torch.empty((world * bs, hidden), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(ref, x)
        if step % 2 == 0:
            out = ag.all_gather_ll(x)
        else:
            out = ag.all_gather_ll_hook(x)()
        torch.cuda.synchronize()
        ag.status.check()
        assert torch.equal(out, ref), f"all-gather mismatch at bs={bs}"
    dist.barrier()


def check_allgather_multicast(rank, world):
    """The same all-gather on a heap bound to an NVLink multicast object: the push is `multimem.st` (one store per 16
    bytes for the whole group). Skipped, on every rank alike, where the GPUs offer no multicast. The heap is closed
    (unmapped, unbound, released) before any rank leaves the check."""
    from dlslime_b200.ops.allgather import AllGatherLLBuffer
    from dlslime_b200.parallel.symm import SymmetricHeap

    hidden = 7168
    slot = (1024 * hidden * 2 + 255) // 256 * 256
    heap = SymmetricHeap(2 * world * slot + 4096, multicast=None)
    if not heap.mc_ptr:
        if rank == 0:
            print("multicast not available here; check skipped", flush=True)
        heap.close()
        dist.barrier()
        return
    try:
        ag = AllGatherLLBuffer(1024, hidden, torch.bfloat16, heap=heap)
        assert ag.use_multicast
        ag._mc_policy = "always"  # every size through the multicast mapping, whatever the size policy would pick
        # the multicast mapping really replicates: a word stored through it shows up in this rank's own region
        for step, bs in enumerate([1, 16, 128, 1024, 16, 1, 1024, 128]):
            x = torch.randn((bs, hidden), device="cuda").to(torch.bfloat16) + rank
            ref = torch.empty((world * bs, hidden), dtype=torch.bfloat16, device="cuda")
            dist.all_gather_into_tensor(ref, x)
            out = ag.all_gather_ll(x) if step % 2 == 0 else ag.all_gather_ll_hook(x)()
            torch.cuda.synchronize()
            ag.status.check()
            assert torch.equal(out, ref), f"multicast all-gather mismatch at bs={bs}"
            dist.barrier()  # nobody starts the step after next (which reuses this half) while a peer still compares
    finally:
        torch.cuda.synchronize()
        dist.barrier()
        heap.close()
        dist.barrier()


def check_alltoall(rank, world):
    from dlslime_b200.ops.alltoall import AllToAllLLBuffer

    hidden, cap = 2048, 256
    a2a = AllToAllLLBuffer(cap, hidden, torch.bfloat16)
    for step, bs in enumerate([1, 16, 256, 16]):
        x = torch.randn((world * bs, hidden), device="cuda").to(torch.bfloat16) + rank
        ref = torch.empty_like(x)
        dist.all_to_all_single(ref, x)
        out = a2a.all_to_all_ll(x) if step % 2 == 0 else a2a.all_to_all_ll_hook(x)()
        torch.cuda.synchronize()
        a2a.status.check()
        assert torch.equal(out, ref), f"all-to-all mismatch at bs={bs}"
        out_t = a2a.all_to_all_ll(x, is_transpose=True)
        torch.cuda.synchronize()
        assert torch.equal(out_t, ref.view(world, bs, hidden).transpose(0, 1)), f"transposed all-to-all mismatch at bs={bs}"
    # variable split: rank r sends (r + p) % 5 rows to rank p
    sizes = [(rank + p) % 5 for p in range(world)]
    offs = torch.tensor([sum(sizes[:p]) for p in range(world + 1)], dtype=torch.int32, device="cuda")
    x = torch.randn((max(sum(sizes), 1), hidden), device="cuda").to(torch.bfloat16)[:sum(sizes)].contiguous()
    recv_sizes = [(s + rank) % 5 for s in range(world)]
    ref = torch.empty((sum(recv_sizes), hidden), dtype=torch.bfloat16, device="cuda")
    dist.all_to_all_single(ref, x, output_split_sizes=recv_sizes, input_split_sizes=sizes)
    data, counts = a2a.all_to_all_ll(x, offsets=offs)
    torch.cuda.synchronize()
    a2a.status.check()
    assert counts.tolist() == recv_sizes, (counts.tolist(), recv_sizes)
    got = torch.cat([data[s, :recv_sizes[s]] for s in range(world)], dim=0)
    assert torch.equal(got, ref), "variable all-to-all mismatch"
    dist.barrier()


def check_moe(rank, world):
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig, init_expert_weights, ref_moe_forward

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    layer = ExpertParallelMoE(cfg, max_tokens=256, seed=7)
    w13, w2 = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=7)
    for step in range(3):
        T = [200, 1, 256, 33, 64, 128, 17, 255][(rank + step) % 8]
        gen = torch.Generator(device="cuda").manual_seed(1000 * step + rank)
        x = torch.randn((T, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((T, cfg.num_experts), generator=gen, device="cuda")
        out = layer(x, lg)
        torch.cuda.synchronize()
        layer.buf.status.check()
        ref, idx, w = ref_moe_forward(cfg, x, lg, w13, w2)
        assert torch.equal(layer.buf.topk_idx[:T].long(), idx)
        err = (out.float() - ref.float()).abs()
        tol = ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5
        assert (err <= tol).all(), f"rank {rank} step {step}: max err {err.max().item()}"
    dist.barrier()


def check_moe_streamed(rank, world):
    """The streamed form (ordered push, per-expert arrival words, gated receive and GEMM as programmatic dependents) on
    real ranks: bit-equal to the regular form on the same inputs, steps of both forms mixed."""
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig, init_expert_weights, ref_moe_forward

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    w = init_expert_weights(cfg, range(rank * (32 // world), (rank + 1) * (32 // world)), "cuda", seed=7)
    plain = ExpertParallelMoE(cfg, max_tokens=256, weights=w)
    fast = ExpertParallelMoE(cfg, max_tokens=256, weights=w, streamed=True)
    w13, w2 = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=7)
    for step in range(5):
        T = [200, 1, 256, 33, 64, 128, 17, 255][(rank + step) % 8]
        gen = torch.Generator(device="cuda").manual_seed(3000 * step + rank)
        x = torch.randn((T, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((T, cfg.num_experts), generator=gen, device="cuda")
        a = plain(x, lg)
        b = fast(x, lg)
        if step == 3:
            b = fast(x, lg)  # twice in a row, no host synchronisation between the steps
        torch.cuda.synchronize()
        fast.buf.status.check()
        assert torch.equal(a, b), f"rank {rank} step {step}: streamed and regular forms differ"
        ref, idx, _ = ref_moe_forward(cfg, x, lg, w13, w2)
        err = (b.float() - ref.float()).abs()
        tol = ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5
        assert (err <= tol).all(), f"rank {rank} step {step}: max err {err.max().item()}"
    dist.barrier()


def check_moe_tbo(rank, world):
    """Two half-batches on two streams: same results as the fp32 oracle, for token counts that split unevenly."""
    from dlslime_b200.models.moe import MoEConfig, TwoBatchOverlapMoE, init_expert_weights, ref_moe_forward

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    layer = TwoBatchOverlapMoE(cfg, max_tokens=256, seed=7)
    w13, w2 = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=7)
    for step in range(4):
        T = [200, 1, 256, 33, 64, 128, 17, 255][(rank + step) % 8]
        gen = torch.Generator(device="cuda").manual_seed(2000 * step + rank)
        x = torch.randn((T, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((T, cfg.num_experts), generator=gen, device="cuda")
        out = layer(x, lg)
        torch.cuda.synchronize()
        layer.check()
        ref, idx, w = ref_moe_forward(cfg, x, lg, w13, w2)
        err = (out.float() - ref.float()).abs()
        tol = ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5
        assert (err <= tol).all(), f"tbo rank {rank} step {step}: max err {err.max().item()}"
    dist.barrier()


def check_ag_gemm(rank, world):
    from dlslime_b200.ops.ag_gemm import AllGatherGemm

    rows, k, n = 256, 1024, 512
    ag = AllGatherGemm(rows, k)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    for step in range(3):
        x = torch.randn(rows, k, device="cuda").to(torch.bfloat16) + rank
        full = torch.empty((world * rows, k), dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(full, x)
        out = ag(x, w)
        torch.cuda.synchronize()
        ag.status.check()
        ref = full.float() @ w.float().t()
        err = (out.float() - ref).abs()
        assert (err <= ref.abs() * 2 ** -7 + ref.abs().mean() * 2 ** -7 + 1e-3).all(), f"ag_gemm rank {rank}: {err.max().item()}"
        dist.barrier()  # nobody may overwrite the gathered matrix before every rank has consumed it


def check_ag_gemm_fp8(rank, world):
    from dlslime_b200.ops import gemm, quant
    from dlslime_b200.ops.ag_gemm import AllGatherGemmFp8

    rows, k, n = 256, 1024, 512
    ag = AllGatherGemmFp8(rows, k)
    wq, sb = quant.fp8_quant_128x128((torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16))
    for step in range(3):
        x = (torch.randn(rows, k, device="cuda") * (1 + rank)).to(torch.bfloat16)
        xq, sx = quant.fp8_quant_1x128(x)
        fq = torch.empty((world * rows, k), dtype=torch.uint8, device="cuda")
        fs = torch.empty((world * rows, k // 128), dtype=torch.float32, device="cuda")
        dist.all_gather_into_tensor(fq, xq.view(torch.uint8))
        dist.all_gather_into_tensor(fs, sx)
        out = ag(x, wq, sb)
        torch.cuda.synchronize()
        ag.status.check()
        ref = gemm.ref_gemm_fp8_blockscaled(fq.view(torch.float8_e4m3fn), fs, wq, sb)
        err = (out.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-3, f"ag_gemm_fp8 rank {rank}: {err}"
        dist.barrier()


def check_torch_backend(rank, world):
    """CUDA tensors through a second process group of the "dlslime" backend: device to device between GPUs (pairs
    r, r ^ 1), producer kernels in front of the send, consumer kernels behind the receive."""
    from datetime import timedelta

    from dlslime_b200 import torch_backend

    # The group object is built the way init_process_group("dlslime") builds it, on a prefix of the default store.
    # (dist.new_group cannot attach a Python process group to a default group that was bound to a device.)
    store = dist.PrefixStore("slime_torch_backend_check", dist.distributed_c10d._get_default_store())
    g = torch_backend._create(store, rank, world, timedelta(seconds=60))
    peer = rank ^ 1
    if peer < world:
        x = torch.randn(1 << 22, device="cuda") * (rank + 1)
        y = torch.empty_like(x)
        ws = [g.send([x], peer, 0), g.recv([y], peer, 0)]
        ws[1].wait(), ws[0].wait()
        z = y * 2  # consumer kernel right behind the receive
        torch.cuda.synchronize()
        sums = torch.stack([x.double().sum(), y.double().sum()]).float()
        allsums = [torch.empty_like(sums) for _ in range(world)]
        dist.all_gather(allsums, sums)  # NCCL, default group
        assert abs(allsums[peer][0].item() - sums[1].item()) <= 1e-3 * max(1.0, abs(sums[1].item())), "payload differs from what the peer sent"
        assert torch.allclose(z, y * 2)
        pg = g if type(g).__name__ == "DirectGroup" else None
        if pg is not None:
            assert pg.counters["direct_sends"] >= 1 and pg.counters["staged_fallbacks"] == 0, pg.counters
    else:
        dist.all_gather([torch.empty(2, device="cuda") for _ in range(world)], torch.zeros(2, device="cuda"))
    dist.barrier()
    g.shutdown()


def check_kv(rank, world):
    """Ranks [0, world/2) play prefill and push into the paged cache of rank + world/2."""
    from dlslime_b200.models.pd_kv import KVShape, PagedKVCache, PrefillSender, wait_layers
    from dlslime_b200.ops._common import default_status
    from dlslime_b200.parallel.symm import SymmetricHeap

    half = world // 2
    shape = KVShape(layers=4)
    lens = [130, 64, 700, 1]
    pages = sum((n + 63) // 64 for n in lens)
    blocks = pages + 9
    heap = SymmetricHeap(PagedKVCache.bytes_needed(shape, blocks))
    is_prefill = rank < half
    owner = rank + half if is_prefill else rank
    cache = PagedKVCache(shape, blocks, heap, owner_rank=owner)
    g = torch.Generator().manual_seed(50 + (rank % half))
    dst_blocks = torch.randperm(blocks, generator=g)[:pages].tolist()
    gen = torch.Generator(device="cuda").manual_seed(70 + (rank % half))
    stage = torch.randn((shape.layers, 2, sum(lens), shape.row), generator=gen, device="cuda").to(shape.dtype)
    dist.barrier()
    if is_prefill:
        sender = PrefillSender(shape, cache, max_tokens=sum(lens), comm_blocks=16)
        sender.plan(lens, dst_blocks)
        sender.kv_stage.copy_(stage)
        d = 256
        hidden = torch.randn(sum(lens), d, device="cuda").to(torch.bfloat16)
        sender.run_prefill_with_transfer(hidden, [(torch.randn(d, d, device="cuda") * 0.05).to(torch.bfloat16)])
        torch.cuda.synchronize()
        default_status().check()
    else:
        assert wait_layers(cache, 1, timeout_s=20.0), "layers did not arrive"
        from dlslime_b200.ops import kv as kvops

        tok_off, blk, ntok = kvops.build_page_tasks(lens, shape.page_tokens, dst_blocks)
        got = cache.tensor()
        for t, b, n in zip(tok_off.tolist(), blk.tolist(), ntok.tolist()):
            assert torch.equal(got[:, :, b, :n], stage[:, :, t:t + n]), "kv page mismatch"
    dist.barrier()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    which = sys.argv[1:] or ["endpoint", "allgather", "allgather_multicast", "alltoall", "moe", "moe_streamed", "moe_tbo", "ag_gemm", "ag_gemm_fp8", "kv", "torch_backend"]
    for name in which:
        globals()[f"check_{name}"](rank, world)
        if rank == 0:
            print(f"CHECK_OK {name}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    print(f"WORKER_OK {rank}", flush=True)


if __name__ == "__main__":
    main()
