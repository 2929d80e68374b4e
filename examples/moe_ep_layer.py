#!/usr/bin/env python3
"""One expert-parallel MoE layer step (dispatch + fp8 quant -> grouped SwiGLU FFN -> combine) on 1..8 GPUs.

    python examples/moe_ep_layer.py                                                       # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/moe_ep_layer.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig  # noqa: E402


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = MoEConfig(num_experts=64, topk=8, hidden=7168, intermediate=2048)
    tokens = 512
    layer = ExpertParallelMoE(cfg, max_tokens=tokens)
    x = torch.randn(tokens, cfg.hidden, device="cuda").to(torch.bfloat16)
    router_logits = torch.randn(tokens, cfg.num_experts, device="cuda")
    y = layer(x, router_logits)          # [tokens, hidden] bf16: sum over the top-k experts, gate-weighted
    torch.cuda.synchronize()
    layer.buf.status.check()
    if int(os.environ.get("RANK", "0")) == 0:
        print("output", tuple(y.shape), y.dtype, "finite:", bool(torch.isfinite(y.float()).all()))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
