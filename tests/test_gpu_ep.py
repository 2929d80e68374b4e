"""Expert-parallel dispatch / expert FFN / combine against the fp32 oracle.

Multi-rank protocols are replayed on ONE GPU: every rank gets its own symmetric
region on the same device and the steps run phase by phase.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_group(world, tokens, cfg, streamed=False):
    from dlslime_b200.models.moe import ExpertParallelMoE, emulated_forward, init_expert_weights, ref_moe_forward
    from dlslime_b200.ops.ep import EpBuffer
    from dlslime_b200.ops._common import default_status

    max_tokens = max(max(tokens), 1)
    bufs = EpBuffer.emulated_group(world, cfg.num_experts, cfg.topk, cfg.hidden, max_tokens)
    layers = [ExpertParallelMoE(cfg, max_tokens, buffer=b, seed=3) for b in bufs]
    w13, w2 = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=3)
    gen = torch.Generator(device="cuda").manual_seed(11)
    for step in range(2):  # two steps: flags and counters must be reusable
        xs = [torch.randn((t, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16) for t in tokens]
        lgs = [torch.randn((t, cfg.num_experts), generator=gen, device="cuda") for t in tokens]
        outs = emulated_forward(layers, xs, lgs, streamed=streamed and step == 1)  # step 0 regular, step 1 streamed: the forms mix
        torch.cuda.synchronize()
        default_status().check()
        for r in range(world):
            if tokens[r] == 0:
                continue
            ref, idx, w = ref_moe_forward(cfg, xs[r], lgs[r], w13, w2)
            got_idx = layers[r].buf.topk_idx[:tokens[r]].long()
            assert torch.equal(got_idx, idx), "top-k selection differs from torch.topk"
            assert torch.allclose(layers[r].buf.topk_w[:tokens[r]], w, rtol=1e-5, atol=1e-7)
            err = (outs[r].float() - ref.float()).abs()
            tol = ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5
            assert (err <= tol).all(), f"rank {r} step {step}: max err {err.max().item()} (ref mean {ref.float().abs().mean().item()})"
        # packed rows: every rank received exactly the rows routed to its experts
        total = sum(int(layers[r].buf.group_offsets[-1].item()) for r in range(world))
        assert total == sum(tokens) * cfg.topk


@pytest.mark.parametrize("world,tokens", [(1, [37]), (2, [17, 3]), (4, [1, 0, 64, 130]), (8, [5, 6, 7, 8, 9, 10, 11, 12])])
def test_moe_layer_emulated_group(world, tokens):
    from dlslime_b200.models.moe import MoEConfig

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    _run_group(world, tokens, cfg)


@pytest.mark.parametrize("world,tokens", [(1, [37]), (2, [17, 3]), (4, [1, 0, 64, 130]), (8, [5, 6, 7, 8, 9, 10, 11, 12])])
def test_moe_layer_emulated_group_streamed(world, tokens):
    """The streamed form (ordered push, per-expert arrival words, gated receive and gated GEMM), replayed rank by rank
    on one stream, against the same oracle; the step before it runs the regular form on the same buffers."""
    from dlslime_b200.models.moe import MoEConfig

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    _run_group(world, tokens, cfg, streamed=True)


def test_streamed_dispatch_lands_the_same_bytes_as_the_regular_one():
    """Both forms of dispatch fill the packed buffers identically: payload, scales, source words, group offsets."""
    from dlslime_b200.ops.ep import EpBuffer
    from dlslime_b200.ops._common import default_status

    world, E, K, H, T = 4, 32, 4, 1024, 70
    gen = torch.Generator(device="cuda").manual_seed(5)
    xs = [torch.randn((T - 9 * r, H), generator=gen, device="cuda").to(torch.bfloat16) for r in range(world)]
    lgs = [torch.randn((x.shape[0], E), generator=gen, device="cuda") for x in xs]
    snaps = []
    for streamed in (False, True):
        bufs = EpBuffer.emulated_group(world, E, K, H, T)
        for b, lg in zip(bufs, lgs):
            (b.route_ordered if streamed else b.route)(lg, lg.shape[0], 1)
        if streamed:
            for b in bufs:
                b.compute_layout(1)
        for b, x in zip(bufs, xs):
            (b.dispatch_ordered if streamed else b.dispatch)(x, 1)
        torch.cuda.synchronize()
        default_status().check()
        snap = []
        for b in bufs:
            rows = int(b.group_offsets[-1].item())
            # rows of one expert land in the order the route kernel's atomics handed out slots, which differs from run
            # to run: compare by source word (experts are contiguous, so sorting by (expert, word) keeps the groups)
            offs = b.group_offsets.tolist()
            expert_of_row = torch.repeat_interleave(torch.arange(len(offs) - 1, device="cuda"),
                                                    torch.tensor([offs[j + 1] - offs[j] for j in range(len(offs) - 1)], device="cuda"))
            info = b.recv_info[:rows]
            order = torch.argsort(expert_of_row * (1 << 52) + info, stable=True)
            snap.append((b.group_offsets.clone(), b.recv_x[:rows].view(torch.uint8)[order].clone(),
                         b.recv_scale[:rows][order].clone(), info[order].clone()))
            if streamed:  # every (source, local expert) word says step 1, and the push counters are back at zero
                arrive = b._view(b.layout.off_arrive, (world, E // world), torch.int64)
                assert bool((arrive == 1).all()) and int(b.pushed.sum().item()) == 0
                assert int(b.push_off[-1].item()) == xs[b.rank].shape[0] * K
        snaps.append(snap)
    for a, b in zip(*snaps):
        for u, v in zip(a, b):
            assert torch.equal(u, v)


@pytest.mark.parametrize("tokens", [1, 96, 512])
def test_streamed_forward_single_rank_three_kernels_at_once(tokens):
    """One real rank: the ordered push, the gated receive and the gated GEMM run at the same time (programmatic
    dependent launches) and must agree with the regular forward (and the oracle) over several steps."""
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig, init_expert_weights, ref_moe_forward

    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    w = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=9)
    plain = ExpertParallelMoE(cfg, tokens, weights=w)
    fast = ExpertParallelMoE(cfg, tokens, weights=w, streamed=True)
    gen = torch.Generator(device="cuda").manual_seed(tokens)
    for step in range(3):
        x = torch.randn((tokens, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((tokens, cfg.num_experts), generator=gen, device="cuda")
        a, b = plain(x, lg), fast(x, lg)
        torch.cuda.synchronize()
        plain.buf.status.check()
        assert torch.equal(a, b), f"step {step}: streamed forward differs from the regular one"
        ref, _, _ = ref_moe_forward(cfg, x, lg, *w)
        err = (b.float() - ref.float()).abs()
        assert (err <= ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5).all()


def test_dispatch_payload_bit_exact():
    """Rows that land in the owner's packed buffer carry exactly the reference fp8 bytes and scales."""
    from dlslime_b200.models.moe import ref_route
    from dlslime_b200.ops.ep import EpBuffer
    from dlslime_b200.ops.quant import ref_quant_1x128
    from dlslime_b200.ops._common import default_status

    world, E, K, H, T = 2, 16, 2, 512, 50
    bufs = EpBuffer.emulated_group(world, E, K, H, T)
    gen = torch.Generator(device="cuda").manual_seed(2)
    xs = [torch.randn((T, H), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(world)]
    lgs = [torch.randn((T, E), generator=gen, device="cuda") for _ in range(world)]
    for b, lg in zip(bufs, lgs):
        b.route(lg, T, 1)
    for b, x in zip(bufs, xs):
        b.dispatch(x, 1)
    torch.cuda.synchronize()
    default_status().check()
    epr = E // world
    for r, b in enumerate(bufs):
        offs = b.group_offsets.tolist()
        info = b.recv_info[:offs[-1]]
        src, slot = (info >> 48).tolist(), (info & ((1 << 48) - 1)).tolist()
        for j in range(epr):
            for row in range(offs[j], offs[j + 1]):
                s, t, k = src[row], slot[row] // K, slot[row] % K
                idx, _ = ref_route(lgs[s], K)
                assert idx[t, k].item() == r * epr + j
                q, sc = ref_quant_1x128(xs[s][t:t + 1])
                assert torch.equal(b.recv_x[row].view(torch.uint8), q[0].view(torch.uint8))
                assert torch.equal(b.recv_scale[row], sc[0])
        # rows of one expert are grouped by source rank in rank order
        for j in range(epr):
            seg = src[offs[j]:offs[j + 1]]
            assert seg == sorted(seg)


def test_wait_times_out_instead_of_hanging():
    """A count row that never arrives makes dispatch give up after its limit and report TIME_OUT."""
    from dlslime_b200.ops.ep import EpBuffer
    from dlslime_b200.ops._common import KernelTimeout, default_status

    bufs = EpBuffer.emulated_group(2, 16, 2, 512, 8, wait_ns=20_000_000)  # 20 ms limit
    x = torch.randn((8, 512), device="cuda").to(torch.bfloat16)
    lg = torch.randn((8, 16), device="cuda")
    bufs[0].route(lg, 8, 1)  # rank 1 never publishes its counts
    bufs[0].dispatch(x, 1)
    torch.cuda.synchronize()
    with pytest.raises(KernelTimeout):
        default_status().check()
    default_status().check()  # the page is cleared after reporting


@pytest.mark.parametrize("tokens", [1, 2, 77, 256])
def test_two_batch_overlap_single_rank(tokens):
    """The two-stream, two-half-batch form of the layer against the fp32 oracle on one rank."""
    from dlslime_b200.models.moe import MoEConfig, TwoBatchOverlapMoE, init_expert_weights, ref_moe_forward

    cfg = MoEConfig(num_experts=16, topk=4, hidden=1024, intermediate=256)
    layer = TwoBatchOverlapMoE(cfg, max_tokens=256, seed=3)
    w13, w2 = init_expert_weights(cfg, range(cfg.num_experts), "cuda", seed=3)
    for step in range(2):
        gen = torch.Generator(device="cuda").manual_seed(31 * tokens + step)
        x = torch.randn((tokens, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((tokens, cfg.num_experts), generator=gen, device="cuda")
        out = layer(x, lg)
        torch.cuda.synchronize()
        layer.check()
        ref, _, _ = ref_moe_forward(cfg, x, lg, w13, w2)
        err = (out.float() - ref.float()).abs()
        tol = ref.float().abs() * 2 ** -6 + ref.float().abs().mean() * 2 ** -5
        assert (err <= tol).all(), f"step {step}: max err {err.max().item()}"


def test_moe_layer_with_fused_dequant_matches_the_two_pass_layer():
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig

    cfg = MoEConfig(num_experts=16, topk=4, hidden=1024, intermediate=256)
    plain = ExpertParallelMoE(cfg, max_tokens=256, seed=5)
    fused = ExpertParallelMoE(cfg, max_tokens=256, weights=(plain.w_gate_up, plain.w_down), fuse_dequant=True)
    for tokens in (1, 77, 256):
        gen = torch.Generator(device="cuda").manual_seed(tokens)
        x = torch.randn((tokens, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16)
        lg = torch.randn((tokens, cfg.num_experts), generator=gen, device="cuda")
        a, b = plain(x, lg), fused(x, lg)
        torch.cuda.synchronize()
        plain.buf.status.check()
        assert torch.equal(a, b), (a.float() - b.float()).abs().max().item()


def test_device_trace_counts_rows_and_waits():
    """The optional trace page: rows pushed per peer add up to tokens x top-k, every waiting kernel reports its calls."""
    from dlslime_b200.models.moe import ExpertParallelMoE, MoEConfig, emulated_forward
    from dlslime_b200.ops.ep import EpBuffer

    world, tokens = 2, [20, 7]
    cfg = MoEConfig(num_experts=32, topk=4, hidden=1024, intermediate=256)
    bufs = EpBuffer.emulated_group(world, cfg.num_experts, cfg.topk, cfg.hidden, max(tokens))
    for b in bufs:
        b.enable_device_trace()
    layers = [ExpertParallelMoE(cfg, max(tokens), buffer=b, seed=3) for b in bufs]
    gen = torch.Generator(device="cuda").manual_seed(4)
    steps = 3
    for _ in range(steps):
        xs = [torch.randn((t, cfg.hidden), generator=gen, device="cuda").to(torch.bfloat16) for t in tokens]
        lgs = [torch.randn((t, cfg.num_experts), generator=gen, device="cuda") for t in tokens]
        emulated_forward(layers, xs, lgs)
    torch.cuda.synchronize()
    for r, b in enumerate(bufs):
        tr = b.device_trace()
        assert sum(p["rows"] for p in tr["peers"]) == steps * tokens[r] * cfg.topk
        assert all(p["steps"] == steps for p in tr["peers"])
        assert tr["peers"][0]["bytes"] == tr["peers"][0]["rows"] * (1024 + 8 * 4 + 8)
        for k in ("dispatch", "receive", "combine"):
            assert tr[k]["calls"] == steps and tr[k]["last_start_ns"] > 0
            assert 0 <= tr[k]["last_wait_ns"] <= tr[k]["total_wait_ns"] < 10**9
    bufs[0].enable_device_trace(False)
    with pytest.raises(RuntimeError):
        bufs[0].device_trace()
