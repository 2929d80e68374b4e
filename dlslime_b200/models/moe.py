"""DeepSeek-V3-shaped expert-parallel MoE layer built from the EP kernels.

One forward step on every rank:

    route -> dispatch (fp8 1x128 quantisation fused with the NVLink push)
          -> receive + dequantise -> grouped gate/up GEMM with SwiGLU epilogue
          -> grouped down GEMM whose epilogue stores rows into the token owners'
             combine buffers over NVLink -> gate-weighted reduction.

``streamed=True`` runs the first half as three kernels at once (programmatic dependent launches in
one stream): the rows are pushed expert by expert, the receive side expands an expert as soon as its rows from every rank
have landed, and the gate/up GEMM's producer waits per expert group, so the tensor cores start on
expert 0 while the later experts are still crossing NVLink.

Expert weights are random N(0, 0.02) bf16 in the ``nn.Linear`` layout. The layer
is the flagship workload of ``bench.py``; ``ref_moe_forward`` is its fp32 PyTorch
oracle.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import gemm
from ..ops.ep import EpBuffer
from ..ops.quant import ref_dequant_1x128, ref_quant_1x128


@dataclass
class MoEConfig:
    num_experts: int = 256
    topk: int = 8
    hidden: int = 7168
    intermediate: int = 2048
    renormalize: bool = False
    init_std: float = 0.02


def init_expert_weights(cfg: MoEConfig, experts: range, device, seed: int = 0):
    """Weights of the given global experts: (w_gate_up [n, 2I, H], w_down [n, H, I]), bf16.

    Expert ``e`` is drawn from its own generator seeded ``seed * 100003 + e`` so a rank's
    shard equals the matching slice of the full set, whatever the world size.
    """
    n = len(experts)
    w13 = torch.empty((n, 2 * cfg.intermediate, cfg.hidden), dtype=torch.bfloat16, device=device)
    w2 = torch.empty((n, cfg.hidden, cfg.intermediate), dtype=torch.bfloat16, device=device)
    gen = torch.Generator(device=device)
    for i, e in enumerate(experts):
        gen.manual_seed(seed * 100003 + e)
        w13[i].copy_(torch.randn((2 * cfg.intermediate, cfg.hidden), generator=gen, device=device, dtype=torch.float32)
                     .mul_(cfg.init_std))
        w2[i].copy_(torch.randn((cfg.hidden, cfg.intermediate), generator=gen, device=device, dtype=torch.float32)
                    .mul_(cfg.init_std))
    return w13, w2


class ExpertParallelMoE:
    """One rank's shard of the MoE layer."""

    def __init__(self, cfg: MoEConfig, max_tokens: int, *, group=None, seed: int = 0, buffer: EpBuffer | None = None,
                 recv_cap: int | None = None, weights=None, thin_waits: bool = False,
                 fuse_dequant: bool = False, streamed: bool = False):
        self.cfg = cfg
        self.buf = buffer or EpBuffer(cfg.num_experts, cfg.topk, cfg.hidden, max_tokens, group=group, recv_cap=recv_cap)
        self.rank, self.world = self.buf.rank, self.buf.world
        dev = self.buf.device
        epr = self.buf.experts_per_rank
        if weights is None:
            weights = init_expert_weights(cfg, range(self.rank * epr, (self.rank + 1) * epr), dev, seed)
        self.w_gate_up, self.w_down = weights
        # thin_waits: every wait for other ranks is a one-block kernel in front of the large kernel, which then starts
        # with its flags already set and never spins (needed when two chains of kernels share the GPU)
        self.thin_waits = thin_waits
        # fuse_dequant: the gate/up GEMM reads the received e4m3 rows and their scales directly and expands them in
        # shared memory (bit-identical to the separate pass, which is then only a one-block wait for the rows). Off by
        # default: with the raw tile next to the bf16 one the ring is 3 stages deep instead of 4 and the expansion sits
        # between the load and the MMA; measured on one GPU the gate/up GEMM takes 3.76 ms instead of 2.73 + 0.13 ms.
        self.fuse_dequant = fuse_dequant
        # streamed: dispatch, receive and the gate/up GEMM run at the same time (see forward_streamed)
        self.streamed = streamed and not fuse_dequant
        # grid of the streamed form's push + receive kernel (0 = three blocks per SM; a multiple of 3)
        import os

        self.comm_blocks = int(os.environ.get("SLIME_EP_COMM_BLOCKS", "0"))
        # words of the gated GEMM's dynamic tile scheduler (SLIME_EP_STATIC_TILES=1: every gridDim-th tile instead)
        self._tile_counter = None if os.environ.get("SLIME_EP_STATIC_TILES") == "1" else torch.zeros(2, dtype=torch.int32, device=dev)
        # pair_gemm: the expert GEMMs on CTA pairs (True: 256 x 256 tiles, "wide": 256 x 512). They win where a local
        # expert sees several hundred rows per step (many ranks), and lose to the single-CTA kernel's 128-row tiles on
        # small groups; SLIME_EP_PAIR_GEMM=0|1|wide overrides the rule, autotune() measures.
        rows_per_expert = max_tokens * cfg.topk * self.world // max(1, cfg.num_experts)
        forced = os.environ.get("SLIME_EP_PAIR_GEMM")
        self.pair_gemm = (rows_per_expert >= 512) if forced is None else {"0": False, "1": True}.get(forced, forced)
        # tile width of the single-CTA expert GEMMs (0 = 256). Narrower tiles were measured for the decode-size step on
        # many ranks (32 experts x 32 rows: 512 tiles = 3.46 waves of the grid) and do not pay: those GEMMs stream weights
        # from HBM, the CTAs do not wait for one another between waves, and a short last wave still fills the memory
        # system (5.66 TB/s of weights with 256-wide tiles, 5.53 with the widths that fill the waves).
        self.tile_n_gate_up = self.tile_n_down = int(os.environ.get("SLIME_EP_TILE_N", "0"))
        # row tiles of 64 where a local expert is expected to see a few dozen rows per step (decode steps): the A part of
        # a pipeline stage halves, the ring gets a fifth stage and more weight bytes are in flight (SLIME_EP_TILE_M=0|64)
        expected = max_tokens * cfg.topk * self.world / max(1, cfg.num_experts)
        forced_m = os.environ.get("SLIME_EP_TILE_M")
        self.tile_m = (64 if expected + 3 * expected ** 0.5 <= 64 else 0) if forced_m is None else int(forced_m)
        cap = self.buf.recv_cap
        self.xd = torch.empty((cap, cfg.hidden), dtype=torch.bfloat16, device=dev)
        self.h = torch.empty((cap, cfg.intermediate), dtype=torch.bfloat16, device=dev)
        self.max_tokens = max_tokens
        self._bases = self.buf.scatter_bases()

    # The steps are separate methods so that a single-GPU test can interleave ranks.
    def step_route(self, logits, T, epoch):
        self.buf.route(logits, T, epoch, self.cfg.renormalize)

    def step_dispatch(self, x, epoch):
        self.buf.dispatch(x, epoch)

    def step_recv(self, T, epoch):
        c = self.cfg
        if self.fuse_dequant:
            self.buf.wait(0, epoch)
            return
        rows = min(self.buf.recv_cap, max(1, 2 * T * c.topk))
        if self.thin_waits:
            self.buf.wait(0, epoch)
        self.buf.recv_dequant(self.xd, epoch, expected_rows=rows)

    def step_gate_up(self):
        if self.fuse_dequant:
            gemm.grouped_gemm_fp8a(self.buf.recv_x, self.buf.recv_scale, self.w_gate_up, self.buf.group_offsets, out=self.h,
                                   epilogue=gemm.EPI_SWIGLU)
            return
        gemm.grouped_gemm_bf16(self.xd, self.w_gate_up, self.buf.group_offsets, out=self.h, epilogue=gemm.EPI_SWIGLU,
                               pair=self.pair_gemm, tile_n=self.tile_n_gate_up, tile_m=self.tile_m)

    def step_down(self):
        c = self.cfg
        gemm.grouped_gemm_bf16(self.h, self.w_down, self.buf.group_offsets, epilogue=gemm.EPI_SCATTER_ROWS,
                               row_info=self.buf.recv_info, scatter_bases=self._bases,
                               scatter_row_bytes=c.hidden * 2, scatter_slots=self.max_tokens * c.topk, pair=self.pair_gemm,
                               tile_n=self.tile_n_down, tile_m=self.tile_m)

    def step_experts(self, T, epoch):
        self.step_recv(T, epoch)
        self.step_gate_up()
        self.step_down()

    def step_combine(self, out, T, epoch, do_signal=True):
        if self.thin_waits and do_signal:
            self.buf.signal(1, epoch)
            self.buf.wait(1, epoch)
            do_signal = False
        self.buf.combine_reduce(out, T, epoch, do_signal=do_signal)

    # -- streamed form: the pieces, so that a single-GPU test can interleave ranks on one stream ---------------------
    def step_route_ordered(self, logits, T, epoch):
        self.buf.route_ordered(logits, T, epoch, self.cfg.renormalize)

    def step_layout(self, epoch):
        self.buf.compute_layout(epoch)

    def step_dispatch_ordered(self, x, epoch, max_blocks=0):
        self.buf.dispatch_ordered(x, epoch, max_blocks=max_blocks)

    def step_recv_gated(self, epoch, max_blocks=0):
        self.buf.recv_dequant_gated(self.xd, epoch, max_blocks=max_blocks)

    def step_gate_up_gated(self, epoch):
        if epoch is None:
            gemm.grouped_gemm_bf16_gated(self.xd, self.w_gate_up, self.buf.group_offsets, self.buf.group_ready,
                                         step_ptr=self.buf.epoch_dev.data_ptr(), out=self.h, epilogue=gemm.EPI_SWIGLU,
                                         trace=self.buf.group_trace, tile_counter=self._tile_counter)
        else:
            gemm.grouped_gemm_bf16_gated(self.xd, self.w_gate_up, self.buf.group_offsets, self.buf.group_ready,
                                         step=epoch, out=self.h, epilogue=gemm.EPI_SWIGLU, trace=self.buf.group_trace,
                                         tile_counter=self._tile_counter)

    def forward_streamed(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """The same layer with dispatch, receive and the gate/up GEMM overlapped.

        Everything is launched into the caller's stream. The ordered push and the gated receive are ONE kernel (two
        pushing blocks and one receiving block per SM); the gated GEMM behind it is its programmatic dependent: it may
        start as soon as every block of that kernel is running, orders itself against the data with the ready words,
        and does not complete before its predecessor has. So push, receive and GEMM share the device without a second
        stream, and a kernel that waits can never keep the kernel it waits for from being scheduled.
        """
        T = x.shape[0]
        if out is None:
            out = torch.empty_like(x)
        self.buf.stage_quantised(x)
        self.step_route_ordered(logits, T, None)
        self.step_layout(None)
        self.buf.stream_comm(T, self.xd, None, self.comm_blocks)
        self.step_gate_up_gated(None)
        self.step_down()
        self.step_combine(out, T, None)
        return out

    def autotune(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None, steps: int = 4) -> dict:
        """Pick the faster expert GEMM (single CTAs or CTA pairs) and then the faster of the two forms of the first half
        (phases one after the other, or streamed) for this shape and world size by running them, and keep both. A form
        replaces the default (single CTAs, phases one after the other) only if it wins by more than 1 %, so that
        run-to-run noise does not pick. Every rank must call this with its own inputs of the step shape; the device times
        are combined as the maximum over ranks, so all ranks decide alike. Which form wins
        depends on the regime: streaming hides the NVLink-bound push under compute-bound expert GEMMs (many ranks, many
        rows per expert) and loses where the GEMMs stream weights from HBM and the extra traffic gets in their way.
        """
        import torch.distributed as dist

        if self.fuse_dequant:
            return {"streamed": False, "reason": "the fused-dequant GEMM has no streamed form"}
        times = {}
        # wide pairs and swapped operands have lost on every shape measured so far (1, 2 and 8 GPUs): they are timed only
        # on request
        import os

        kinds = {"single": False, "pair": True}
        if os.environ.get("SLIME_EP_AUTOTUNE_ALL") == "1":
            kinds.update({"wide": "wide", "swap": "swap"})
        for form in (*kinds, True):
            if form is True:
                best = min(kinds, key=lambda k: times[k])
                if times[best] > 0.99 * times["single"]:
                    best = "single"
                self.pair_gemm = kinds[best]
                times[False] = times[best]
            self.streamed = form is True
            if form is not True:
                self.pair_gemm = kinds[form]
            for _ in range(2):
                self.forward(x, logits, out)
            if dist.is_initialized():
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                self.forward(x, logits, out)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / steps], device=x.device, dtype=torch.float64)
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times[form] = float(t.item())
            self.buf.status.check()
        self.streamed = times[True] < 0.99 * times[False]
        return {"streamed": self.streamed, "pair_gemm": self.pair_gemm, "serial_ms": round(times[False], 4),
                "serial_single_cta_ms": round(times["single"], 4), "serial_cta_pair_ms": round(times["pair"], 4),
                **({"serial_cta_pair_wide_ms": round(times["wide"], 4), "serial_cta_pair_swapped_ms": round(times["swap"], 4)}
                   if "wide" in times else {}),
                "streamed_ms": round(times[True], 4)}

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [T, hidden] bf16, router logits [T, num_experts] fp32 -> [T, hidden] bf16."""
        if self.streamed:
            return self.forward_streamed(x, logits, out)
        T = x.shape[0]
        if out is None:
            out = torch.empty_like(x)
        # epoch=None: the step counter lives on the device, so this sequence of launches is graph-capturable
        self.step_route(logits, T, None)
        self.step_dispatch(x, None)
        self.step_experts(T, None)
        self.step_combine(out, T, None)
        return out

    __call__ = forward

    def capture(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """Capture one forward on fixed buffers into a CUDA graph (decode-size steps are launch-bound).

        ``x``, ``logits`` and ``out`` become the graph's static input / output buffers: copy new inputs into
        them and call ``graph.replay()``. Runs two eager warm-up steps first, on every rank alike.
        """
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self.forward(x, logits, out)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward(x, logits, out)
        return graph


class TwoBatchOverlapMoE:
    """The same layer with the step split into two half-batches on two streams, so that the communication phases
    of one half (dispatch, receive, combine: NVLink- and HBM-bound) run while the tensor cores work on the other
    half's expert GEMMs.

    The halves are two :class:`ExpertParallelMoE` instances that share the expert weights and own their
    symmetric buffers and step counters, so no protocol state is shared and the two chains never wait on each other.
    Waits for other ranks are one-block kernels in front of the large kernels (``thin_waits``): a large grid that spins
    could fill the GPU while the block that has to signal for the OTHER chain cannot be scheduled, on two ranks in
    opposite order, and then neither would ever be released (seen as 1 s timeouts on two GPUs at full size).
    """

    def __init__(self, cfg: MoEConfig, max_tokens: int, *, group=None, seed: int = 0, weights=None):
        half = (max_tokens + 1) // 2
        self.cfg, self.max_tokens, self.half = cfg, max_tokens, half
        self.a = ExpertParallelMoE(cfg, half, group=group, seed=seed, weights=weights, thin_waits=True)
        self.b = ExpertParallelMoE(cfg, half, group=group, weights=(self.a.w_gate_up, self.a.w_down), thin_waits=True)
        self.rank, self.world = self.a.rank, self.a.world
        self.buf = self.a.buf  # status page and geometry for callers that look at the single-batch layer's buffer
        self.w_gate_up, self.w_down = self.a.w_gate_up, self.a.w_down
        self.sa, self.sb = torch.cuda.Stream(), torch.cuda.Stream()
        self._fork, self._ja, self._jb = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()

    def forward(self, x: torch.Tensor, logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        T = x.shape[0]
        if out is None:
            out = torch.empty_like(x)
        t0 = (T + 1) // 2
        parts = [(self.a, self.sa, slice(0, t0)), (self.b, self.sb, slice(t0, T))]
        cur = torch.cuda.current_stream()
        self._fork.record(cur)
        for _, s, _ in parts:
            s.wait_event(self._fork)
        # issue order = the order in which every rank's kernels appear: both dispatches first, then the expert phases
        for layer, s, sl in parts:
            with torch.cuda.stream(s):
                n = sl.stop - sl.start
                layer.step_route(logits[sl], n, None)
                layer.step_dispatch(x[sl], None)
        for layer, s, sl in parts:
            with torch.cuda.stream(s):
                layer.step_experts(sl.stop - sl.start, None)
        for layer, s, sl in parts:
            with torch.cuda.stream(s):
                layer.step_combine(out[sl], sl.stop - sl.start, None)
        self._ja.record(self.sa)
        self._jb.record(self.sb)
        cur.wait_event(self._ja)
        cur.wait_event(self._jb)
        return out

    __call__ = forward

    def check(self) -> None:
        self.a.buf.status.check()
        self.b.buf.status.check()


def emulated_forward(layers: list[ExpertParallelMoE], xs, logits, streamed: bool = False):
    """Run one step of a whole emulated group on one GPU, phase by phase (``streamed``: through the kernels of the
    streamed form, one after the other on one stream, so every wait finds its word already set)."""
    outs = [torch.empty_like(x) for x in xs]
    epochs = [layer.buf.next_epoch() for layer in layers]
    if streamed:
        for layer, x, lg, e in zip(layers, xs, logits, epochs):
            layer.step_route_ordered(lg, x.shape[0], e)
        for layer, e in zip(layers, epochs):
            layer.step_layout(e)
        for layer, x, e in zip(layers, xs, epochs):
            layer.step_dispatch_ordered(x, e)
        for layer, e in zip(layers, epochs):
            layer.step_recv_gated(e)
            layer.step_gate_up_gated(e)
            layer.step_down()
    else:
        for layer, x, lg, e in zip(layers, xs, logits, epochs):
            layer.step_route(lg, x.shape[0], e)
        for layer, x, e in zip(layers, xs, epochs):
            layer.step_dispatch(x, e)
        for layer, x, e in zip(layers, xs, epochs):
            layer.step_experts(x.shape[0], e)
    for layer, e in zip(layers, epochs):
        layer.buf.signal(1, e)
    for layer, x, out, e in zip(layers, xs, outs, epochs):
        layer.step_combine(out, x.shape[0], e, do_signal=False)
    return outs


def ref_route(logits: torch.Tensor, topk: int, renormalize: bool = False):
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, topk, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return idx, w


def ref_moe_forward(cfg: MoEConfig, x: torch.Tensor, logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor):
    """fp32 restatement of the layer for ALL experts held in one place.

    Mirrors the roundings of the kernels: fp8 1x128 quantisation of the token,
    bf16 dequantised activations, bf16 intermediate and expert outputs, fp32
    gate-weighted sum rounded once to bf16.
    """
    idx, w = ref_route(logits, cfg.topk, cfg.renormalize)
    q, s = ref_quant_1x128(x)
    xd = ref_dequant_1x128(q, s).to(torch.bfloat16).float()
    out = torch.zeros_like(xd)
    inter = cfg.intermediate
    for e in range(cfg.num_experts):
        sel = (idx == e)
        tok = sel.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        xe = xd[tok]
        g = xe @ w_gate_up[e, :inter].float().t()
        u = xe @ w_gate_up[e, inter:].float().t()
        h = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float()
        y = (h @ w_down[e].float().t()).to(torch.bfloat16).float()
        gate = (w[tok] * sel[tok]).sum(-1, keepdim=True)
        out[tok] += gate * y
    return out.to(torch.bfloat16), idx, w
