"""Reference arm of bench.py: the same MoE-layer step composed from the UNMODIFIED reference package.

The reference (installed under ``baseline/_ref``) ships no kernels and no dispatch / combine op. What
a user of it has is ``NVLinkEndpoint.read`` (one ``cudaMemcpyAsync`` per assignment, read only), so the
step is composed the way such a user would: torch for routing, fp8 block quantisation, sorting by
expert, the grouped SwiGLU FFN and the weighted sum (``baseline/torch_moe.py``); NCCL for the count
exchange and the barriers; the reference endpoint for every token row that crosses GPUs, pulled by the
receiving rank. Nothing from the ``dlslime_b200`` package is imported here or by anything this imports.

With one GPU nothing crosses ranks: the reference package is loaded and its endpoint registers the arena,
but it has nothing to read (it cannot map memory of its own process), so the local segments are plain
device copies; the result says so (``reference_package_used``).
"""

from __future__ import annotations

import os
import sys

from .torch_moe import E, HIDDEN, TOPK, ExpertFFN, combine, dequant_1x128, init_weights, quant_1x128, route


def _load_reference():
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    from dlslime import _slime_c  # the reference's own extension module

    return _slime_c


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
        w13, w2 = init_weights(range(rank * self.epr, (rank + 1) * self.epr), dev)
        self.ffn = ExpertFFN(w13, w2)
        self.counts_all = torch.empty((world, E), dtype=torch.int64, device=dev)
        self.copies = 0
        self.peers = {}
        ref = _load_reference()
        exporter = ref.NVLinkEndpoint()
        exporter.register_memory_region(self.arena.data_ptr(), 0, total, "arena")
        self._exporter = exporter
        if world > 1:
            infos = [None] * world
            dist.all_gather_object(infos, exporter.endpoint_info())
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
        w, idx = route(logits)
        q, scale = quant_1x128(x)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        tok = order // TOPK
        torch.index_select(q, 0, tok, out=self.send_q)
        torch.index_select(scale, 0, tok, out=self.send_s)
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
        so, eo, sp, mn = send_off.tolist(), exp_off.tolist(), src_prefix.tolist(), mine.tolist()
        for s in range(W):
            pairs = [(so[s][self.rank * epr + j], eo[j] + sp[s][j], mn[s][j]) for j in range(epr)]
            self._pull(s, "recv_q", self.recv_q, "send_q", self.send_q, pairs, HIDDEN)
            self._pull(s, "recv_s", self.recv_s, "send_s", self.send_s, pairs, HIDDEN // 128 * 4)
        R = eo[-1]
        xd = dequant_1x128(self.recv_q[:R], self.recv_s[:R])
        offs_host = exp_off[1:].to(torch.int32)
        self.y[:R].copy_(self.ffn(xd, offs_host.to(x.device, non_blocking=True), offs_host))
        if W > 1:
            dist.barrier()  # every rank's expert outputs are complete before anyone pulls them back
        # combine: my sorted rows of expert e live on rank e // epr at (its exp_off[e % epr] + its src_prefix[me, e % epr])
        my_off = so[self.rank]
        for p in range(W):
            cols = c[:, p * epr:(p + 1) * epr]
            p_exp_off = torch.cat([torch.zeros(1, dtype=torch.int64), cols.sum(0).cumsum(0)]).tolist()
            p_prefix = torch.cat([torch.zeros(1, epr, dtype=torch.int64), cols.cumsum(0)], 0).tolist()
            colsl = cols.tolist()
            pairs = [(p_exp_off[j] + p_prefix[self.rank][j], my_off[p * epr + j], colsl[self.rank][j]) for j in range(epr)]
            self._pull(p, "ret", self.ret, "y", self.y, pairs, HIDDEN * 2)
        combine(self.ret, order, w, out)
        if W > 1:
            dist.barrier()  # nobody may refill its send / result buffers while a peer still reads them
        return out


def run(args, rank, world, local, T, Harness):
    try:
        layer = ReferenceMoE(rank, world, T)
    except Exception as e:  # the reference failed to import or to map peer memory
        return {"unavailable": f"reference endpoint could not be set up: {type(e).__name__}: {e}"[:300]}
    h = Harness(layer.forward, T, rank, world, local, args, pipelined=args.mode == "normal")
    res = h.run_all()
    layer.copies = 0
    layer.forward(h.dev_x[0], h.dev_lg[0], h.out)
    res.update({
        "launches": 0, "weights_gb": (layer.ffn.w13.numel() + layer.ffn.w2.numel()) * 2 / 1e9,
        "reference_package_used": world > 1,
        "check": h.check(layer.forward),
        "notes": {"reference_endpoint_copies_per_step": layer.copies, "expert_ffn": layer.ffn.mode,
                  "transport": "reference NVLinkEndpoint.read" if world > 1 else
                  "local device copies (one GPU: nothing crosses ranks; the reference endpoint is loaded and holds the arena)"}})
    return res
