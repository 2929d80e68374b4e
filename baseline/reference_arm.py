"""Reference arm of bench.py: the same MoE-layer step composed from the UNMODIFIED reference package.

The reference (installed under ``baseline/_ref``) ships no kernels and no dispatch / combine op. What
a user of it has is ``NVLinkEndpoint.read`` (one ``cudaMemcpyAsync`` per assignment, read only), so the
step is composed the way such a user would: torch for routing, fp8 block quantisation, sorting by
expert, the per-expert SwiGLU FFN (cuBLAS) and the weighted sum; NCCL for the count exchange and the
barriers; the reference endpoint for every token row that crosses GPUs, pulled by the receiving rank.
Nothing from the ``dlslime_b200`` package is imported here.

With one GPU nothing crosses ranks and the reference endpoint has nothing to do (it cannot map memory
of its own process); the local segments are then plain device copies, which the result records.
"""

from __future__ import annotations

import os
import sys

E, TOPK, HIDDEN, INTER = 256, 8, 7168, 2048
FP8_MAX = 448.0


def _load_reference():
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    from dlslime import _slime_c  # the reference's own extension module

    return _slime_c


def _init_weights(experts, device, seed=0):
    import torch

    w13 = torch.empty((len(experts), 2 * INTER, HIDDEN), dtype=torch.bfloat16, device=device)
    w2 = torch.empty((len(experts), HIDDEN, INTER), dtype=torch.bfloat16, device=device)
    gen = torch.Generator(device=device)
    for i, e in enumerate(experts):
        gen.manual_seed(seed * 100003 + e)
        w13[i].copy_(torch.randn((2 * INTER, HIDDEN), generator=gen, device=device).mul_(0.02))
        w2[i].copy_(torch.randn((HIDDEN, INTER), generator=gen, device=device).mul_(0.02))
    return w13, w2


class ReferenceMoE:
    def __init__(self, rank, world, T):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.rank, self.world, self.T = rank, world, T
        self.epr = E // world
        dev = torch.device("cuda", torch.cuda.current_device())
        n = T * TOPK
        cap = world * n  # worst case rows this rank can receive
        # Every buffer a peer touches lives in ONE arena that is the first allocation of the process, hence
        # a cudaMalloc segment of its own: the reference opens an IPC handle once per allocation and adds
        # offsets to the allocation's base, so regions must start at a base and share no allocation.
        spec = [("send_q", (n, HIDDEN), torch.uint8), ("send_s", (n, HIDDEN // 128), torch.float32),
                ("recv_q", (cap, HIDDEN), torch.uint8), ("recv_s", (cap, HIDDEN // 128), torch.float32),
                ("y", (cap, HIDDEN), torch.bfloat16), ("ret", (n, HIDDEN), torch.bfloat16)]
        self.off, total = {}, 0
        for name, shape, dt in spec:
            self.off[name] = total
            total += (shape[0] * shape[1] * torch.empty((), dtype=dt).element_size() + 255) // 256 * 256
        total = max(total, 32 << 20)
        self.arena = torch.empty(total, dtype=torch.uint8, device=dev)
        bases = {seg["address"] for seg in torch.cuda.memory_snapshot()}
        if self.arena.data_ptr() not in bases:
            raise RuntimeError("the arena is not at the base of a CUDA allocation; refusing to export it")
        for name, shape, dt in spec:
            nbytes = shape[0] * shape[1] * torch.empty((), dtype=dt).element_size()
            setattr(self, name, self.arena[self.off[name]:self.off[name] + nbytes].view(dt).view(shape))
        self.w13, self.w2 = _init_weights(range(rank * self.epr, (rank + 1) * self.epr), dev)
        self.counts_all = torch.empty((world, E), dtype=torch.int64, device=dev)
        self.copies = 0
        self.peers = {}
        if world > 1:
            ref = _load_reference()
            exporter = ref.NVLinkEndpoint()
            exporter.register_memory_region(self.arena.data_ptr(), 0, total, "arena")
            infos = [None] * world
            dist.all_gather_object(infos, exporter.endpoint_info())
            self._exporter = exporter
            # one endpoint per peer (the reference's model is one endpoint per connection); each peer's
            # handle is opened exactly once in this process
            for p in range(world):
                if p == rank:
                    continue
                ep = ref.NVLinkEndpoint()
                ep.register_memory_region(self.arena.data_ptr(), 0, total, "arena")
                ep.connect(infos[p])
                self.peers[p] = ep
            dist.barrier()

    def _pull(self, p, local_name, local_t, remote_name, remote_t, pairs, row_bytes):
        """pairs: (remote_row, local_row, rows). Remote reads go through the reference endpoint."""
        if p == self.rank:
            for r, l, n in pairs:
                if n > 0:
                    local_t[l:l + n].copy_(remote_t[r:r + n])
            return
        lo, ro = self.off[local_name], self.off[remote_name]
        assign = [("arena", "arena", ro + r * row_bytes, lo + l * row_bytes, n * row_bytes) for r, l, n in pairs if n > 0]
        if assign:
            self.peers[p].read(assign, None)
            self.copies += len(assign)

    def forward(self, x, logits, out):
        torch, dist = self.torch, self.dist
        T, W, epr = x.shape[0], self.world, self.epr
        probs = torch.softmax(logits.float(), dim=-1)
        w, idx = torch.topk(probs, TOPK, dim=-1)
        xf = x.float().view(T, HIDDEN // 128, 128)
        scale = xf.abs().amax(-1).clamp_min(1e-4) / FP8_MAX
        q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn).view(T, HIDDEN)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        tok = order // TOPK
        self.send_q.copy_(q.view(torch.uint8)[tok])
        self.send_s.copy_(scale[tok])
        counts = torch.bincount(flat, minlength=E)
        if W > 1:
            dist.all_gather_into_tensor(self.counts_all, counts)
        else:
            self.counts_all.copy_(counts.unsqueeze(0))
        c = self.counts_all.cpu()  # the host drives every copy, so it needs the counts
        send_off = torch.cat([torch.zeros(W, 1, dtype=torch.int64), c.cumsum(1)], 1)  # [W, E+1] row offsets in each sender's buffer
        mine = c[:, self.rank * epr:(self.rank + 1) * epr]  # [W, epr]
        per_expert = mine.sum(0)
        exp_off = torch.cat([torch.zeros(1, dtype=torch.int64), per_expert.cumsum(0)])
        # dispatch: rows of expert j from source s land at exp_off[j] + sum_{s'<s} mine[s', j]
        src_prefix = torch.cat([torch.zeros(1, epr, dtype=torch.int64), mine.cumsum(0)], 0)
        for s in range(W):
            pairs = [(int(send_off[s, self.rank * epr + j]), int(exp_off[j] + src_prefix[s, j]), int(mine[s, j])) for j in range(epr)]
            self._pull(s, "recv_q", self.recv_q, "send_q", self.send_q, pairs, HIDDEN)
            self._pull(s, "recv_s", self.recv_s, "send_s", self.send_s, pairs, HIDDEN // 128 * 4)
        R = int(exp_off[-1])
        xd = (self.recv_q[:R].view(torch.float8_e4m3fn).float().view(R, HIDDEN // 128, 128) * self.recv_s[:R].unsqueeze(-1)).view(R, HIDDEN).to(torch.bfloat16)
        for j in range(epr):
            a, b = int(exp_off[j]), int(exp_off[j + 1])
            if b > a:
                gu = xd[a:b] @ self.w13[j].t()
                h = torch.nn.functional.silu(gu[:, :INTER]) * gu[:, INTER:]
                torch.matmul(h, self.w2[j].t(), out=self.y[a:b])
        if W > 1:
            dist.barrier()  # every rank's expert outputs are complete before anyone pulls them back
        # combine: my sorted rows of expert e live on rank e // epr at (its exp_off[e % epr] + its src_prefix[me, e % epr])
        my_off = send_off[self.rank]
        for p in range(W):
            cols = c[:, p * epr:(p + 1) * epr]
            p_exp_off = torch.cat([torch.zeros(1, dtype=torch.int64), cols.sum(0).cumsum(0)])
            p_prefix = torch.cat([torch.zeros(1, epr, dtype=torch.int64), cols.cumsum(0)], 0)
            pairs = [(int(p_exp_off[j] + p_prefix[self.rank, j]), int(my_off[p * epr + j]), int(cols[self.rank, j])) for j in range(epr)]
            self._pull(p, "ret", self.ret, "y", self.y, pairs, HIDDEN * 2)
        unsorted = torch.empty_like(self.ret)
        unsorted[order] = self.ret
        out.copy_((unsorted.view(T, TOPK, HIDDEN).float() * w.unsqueeze(-1)).sum(1))
        if W > 1:
            dist.barrier()  # nobody may refill its send / result buffers while a peer still reads them
        return out


def run(args, rank, world, local, T, make_inputs, sync_all, max_over_ranks, ClockSampler):
    import torch

    try:
        layer = ReferenceMoE(rank, world, T)
    except Exception as e:  # the reference failed to import or to map peer memory
        return {"unavailable": f"reference endpoint could not be set up: {type(e).__name__}: {e}"[:300]}
    n_in = min(4, max(1, args.steps))
    host_x, host_lg = make_inputs(T, rank, n_in)
    dev_x = [h.cuda() for h in host_x]
    dev_lg = [h.cuda() for h in host_lg]
    out = torch.empty((T, HIDDEN), dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty((T, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x_stage, lg_stage = torch.empty_like(dev_x[0]), torch.empty_like(dev_lg[0])

    def step_device(i):
        layer.forward(dev_x[i % n_in], dev_lg[i % n_in], out)

    def step_e2e(i):
        x_stage.copy_(host_x[i % n_in], non_blocking=True)
        lg_stage.copy_(host_lg[i % n_in], non_blocking=True)
        layer.forward(x_stage, lg_stage, out)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn):
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        for i in range(args.warmup):
            fn(i)
        sync_all(world)
        sampler.mark_begin()
        layer.copies = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        sync_all(world)
        sampler.mark_end()
        clocks = sampler.stop() if rank == 0 else None
        return max_over_ranks(e0.elapsed_time(e1) / args.steps, world), clocks

    ms_dev, clocks = timed(step_device)
    copies = layer.copies
    ms_e2e, _ = timed(step_e2e)
    remote = (world - 1) / world
    nv_bytes = T * TOPK * (HIDDEN + HIDDEN // 128 * 4) * remote + T * TOPK * HIDDEN * 2 * remote
    return {"ms_dev": ms_dev, "ms_e2e": ms_e2e, "clocks": clocks, "T": T, "h2d": host_x[0].numel() * 2 + host_lg[0].numel() * 4,
            "d2h": host_out.numel() * 2, "launches": 0, "weights_gb": (layer.w13.numel() + layer.w2.numel()) * 2 / 1e9,
            "nvlink_bytes_per_rank": nv_bytes,
            "breakdown_us": {"reference_endpoint_copies_per_run": copies,
                             "transport": "reference NVLinkEndpoint.read" if world > 1 else "local device copies (one GPU: nothing crosses ranks)"}}
