"""Tuned library composite of bench.py (``--impl tuned``): the same MoE-layer step from stock PyTorch + NCCL only.

This is what a careful user without this repository's kernels (and without the reference's endpoint) would write:
NCCL ``all_to_all_single`` with exact split sizes for the fp8 payload, the scales and the expert outputs, one
grouped GEMM per projection (``torch.nn.functional.grouped_mm``), bf16 dequantisation without fp32 temporaries, and
one host synchronisation per step (the split sizes of an unpadded all-to-all have to be known on the host). It is
an extra line beside the reference arm, there to show the margin against well-used libraries; nothing from the
``dlslime_b200`` package or from the reference is imported.
"""

from __future__ import annotations

from .torch_moe import E, HIDDEN, TOPK, ExpertFFN, combine, dequant_1x128, init_weights, quant_1x128, route


class TunedMoE:
    def __init__(self, rank, world, T):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.rank, self.world, self.T = rank, world, T
        self.epr = E // world
        dev = torch.device("cuda", torch.cuda.current_device())
        w13, w2 = init_weights(range(rank * self.epr, (rank + 1) * self.epr), dev)
        self.ffn = ExpertFFN(w13, w2)
        self.counts_in = torch.empty((world, self.epr), dtype=torch.int64, device=dev)
        self.local_expert = torch.arange(self.epr, device=dev).repeat(world)  # expert of each (source, expert) block

    def forward(self, x, logits, out):
        torch, dist = self.torch, self.dist
        T, W, epr = x.shape[0], self.world, self.epr
        w, idx = route(logits)
        q, scale = quant_1x128(x)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)  # rows sorted by global expert = by destination rank, then local expert
        tok = order // TOPK
        send_q = q.index_select(0, tok)
        send_s = scale.index_select(0, tok)
        counts = torch.bincount(flat, minlength=E).view(W, epr)
        if W > 1:
            dist.all_to_all_single(self.counts_in, counts)  # [source, local expert]
            both = torch.stack([counts.sum(1), self.counts_in.sum(1)]).cpu()  # the one host sync: split sizes
            in_split, out_split = both[0].tolist(), both[1].tolist()
            R = sum(out_split)
            recv_q = torch.empty((R, HIDDEN), dtype=torch.uint8, device=x.device)
            recv_s = torch.empty((R, HIDDEN // 128), dtype=torch.float32, device=x.device)
            dist.all_to_all_single(recv_q, send_q, out_split, in_split)
            dist.all_to_all_single(recv_s, send_s, out_split, in_split)
            # received rows are (source, local expert)-major; the grouped GEMM wants local-expert-major
            blocks = self.counts_in.reshape(-1)
            row_expert = torch.repeat_interleave(self.local_expert, blocks, output_size=R)
            perm = torch.argsort(row_expert, stable=True)
            offs = self.counts_in.sum(0).cumsum(0).to(torch.int32)
            xd = dequant_1x128(recv_q.index_select(0, perm), recv_s.index_select(0, perm))
            y_sorted = self.ffn(xd, offs)
            y = torch.empty_like(y_sorted)
            y[perm] = y_sorted
            ret = torch.empty((T * TOPK, HIDDEN), dtype=torch.bfloat16, device=x.device)
            dist.all_to_all_single(ret, y, in_split, out_split)
        else:
            offs = counts.view(-1).cumsum(0).to(torch.int32)
            ret = self.ffn(dequant_1x128(send_q, send_s), offs)
        return combine(ret, order, w, out)


def run(args, rank, world, local, T, Harness):
    layer = TunedMoE(rank, world, T)
    h = Harness(layer.forward, T, rank, world, local, args, pipelined=args.mode == "normal")
    res = h.run_all()
    res.update({"launches": 0, "weights_gb": (layer.ffn.w13.numel() + layer.ffn.w2.numel()) * 2 / 1e9,
                "check": h.check(layer.forward),
                "notes": {"expert_ffn": layer.ffn.mode, "transport": "NCCL all_to_all_single" if world > 1 else "none (one GPU)"}})
    return res
