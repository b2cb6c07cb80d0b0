"""Batched decode loop of a Qwen3-Next-like hybrid model around the MoE path of this library.

Upstream's ``ModelRunner`` decodes one sequence at a time and pins its linear-attention path
to 256 experts / top-8 (``src/model.rs:277-282,413-415,1452-1538``), so the batched
configuration (48 layers, three GatedDeltaNet layers to one gated-attention layer, batch 128,
4096-token context, 512 experts top-10 + shared expert in NVFP4) needs a host loop of its own.
This is that loop. What runs through the C ABI of this library, per layer:

    residual add + RMSNorm + NVFP4 quantisation of the tokens   qs3_fused_add_rmsnorm_nvfp4
    router GEMM, top-k, experts, shared expert, combine,
    residual add + the next layer's input norm                  qs3_moe_layer_execute

and once per step the first norm (``qsfi_rmsnorm``) and the LM head (``qscb_gemm_bf16``).
The token mixers (gated attention over a KV cache, GatedDeltaNet recurrence) are NOT part of
this library: they are stand-ins written with torch operators, with the tensor shapes, state
sizes and memory traffic of the real layers, so that the step time the MoE share is quoted
against is a realistic one. The KV cache is paged: fixed-size pages in a pool, addressed through a
CSR page table as upstream's runtime builds it (src/runtime.rs:99-181). One step is captured in a
CUDA graph and replayed.

``python -m qs3_b200.hybrid_decode`` prints one JSON line: decode tokens/s and the share of the
step spent in the calls of this library.
"""
from __future__ import annotations

import argparse
import json
import math
from dataclasses import dataclass, replace

import torch

from . import capi, ops


@dataclass(frozen=True)
class HybridConfig:
    layers: int = 48
    attention_every: int = 4         # layers 3, 7, 11, ... are attention, the rest GatedDeltaNet
    hidden: int = 2048
    vocab: int = 151936
    # gated attention
    q_heads: int = 16
    kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    # GatedDeltaNet
    gdn_v_heads: int = 32
    gdn_qk_heads: int = 16
    gdn_head_dim: int = 128
    conv_kernel: int = 4
    # MoE block
    experts: int = 512
    top_k: int = 10
    inter: int = 512
    shared_inter: int = 512
    # workload
    batch: int = 128
    context: int = 4096
    new_tokens: int = 256
    page_size: int = 16              # tokens per KV-cache page
    eps: float = 1e-6
    seed: int = 0

    def is_attention(self, layer: int) -> bool:
        return layer % self.attention_every == self.attention_every - 1

    def moe_weight_bytes_per_layer(self) -> int:
        """NVFP4 bytes of one layer's routed + shared experts (codes + e4m3 scales)."""
        per_elem = 9 / 16
        routed = self.experts * 3 * self.inter * self.hidden * per_elem
        shared = 3 * self.shared_inter * self.hidden * per_elem
        return int(routed + shared)


def tiny_config(**kw) -> HybridConfig:
    """A configuration small enough for a parity test (same structure, small sizes)."""
    base = HybridConfig(layers=4, hidden=256, vocab=512, q_heads=4, kv_heads=2, head_dim=64, rotary_dim=16,
                        gdn_v_heads=4, gdn_qk_heads=2, gdn_head_dim=32, experts=16, top_k=2, inter=256,
                        shared_inter=256, batch=8, context=24, new_tokens=4)
    return replace(base, **kw)


def _normal(shape, std, gen, dev, dtype=torch.bfloat16, chunk=1 << 26):
    """N(0, std) tensor generated in chunks (the f32 staging of a whole expert tensor would
    double its footprint)."""
    out = torch.empty(shape, dtype=dtype, device=dev)
    flat = out.view(-1)
    for a in range(0, flat.numel(), chunk):
        b = min(a + chunk, flat.numel())
        flat[a:b] = (torch.randn(b - a, generator=gen, device=dev, dtype=torch.float32) * std).to(dtype)
    return out


class _MoeBlock:
    """Weights of one layer's MoE block, NVFP4."""

    def __init__(self, ctx, cfg: HybridConfig, gen, dev, keep_linear_scales=False):
        h, i, e, s = cfg.hidden, cfg.inter, cfg.experts, cfg.shared_inter
        # the linear-layout block scales are only needed by a CPU check of the block
        q = lambda shape, gated: ops.nvfp4_quantize_weight(ctx, _normal(shape, 0.02, gen, dev), gated,
                                                           linear=keep_linear_scales)
        self.router = _normal((e, h), 0.02, gen, dev)
        self.gate_up = q((e, 2 * i, h), True)
        self.down = q((e, h, i), False)
        self.shared = ops.SharedExpert(q((1, 2 * s, h), True), q((1, h, s), False), _normal((1, h), 0.02, gen, dev), s)
        self.post_mixer_norm = torch.ones(h, dtype=torch.bfloat16, device=dev)


class _Attention:
    """Stand-in for a gated-attention layer (torch operators): q/k/v projections with an output
    gate, per-head RMS norm of q and k, rotary embedding on the first `rotary_dim` dimensions,
    attention of the new token over a PAGED KV cache, output projection.

    The cache is a pool of fixed-size pages [pages, kv_heads, page_size, head_dim] addressed through a
    CSR page table, as upstream's runtime lays it out (src/runtime.rs:99-181: `kv_indptr` [batch + 1]
    into `kv_indices` [pages of all sequences]); pages are handed out in a shuffled order so that the
    indirection is real. Every step looks its pages up (a gather of the sequence's pages) and writes
    the new token's K and V into slot `pos % page_size` of page `kv_indices[kv_indptr[b] + pos // page_size]`."""

    def __init__(self, cfg: HybridConfig, gen, dev, max_len):
        h, qh, kvh, d = cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim
        self.cfg = cfg
        self.w_qg = _normal((2 * qh * d, h), 0.02, gen, dev)       # query and output gate
        self.w_kv = _normal((2 * kvh * d, h), 0.02, gen, dev)
        self.w_o = _normal((h, qh * d), 0.02, gen, dev)
        self.page = cfg.page_size
        self.pages_per_seq = (max_len + self.page - 1) // self.page
        pages = cfg.batch * self.pages_per_seq
        self.kv_indptr = torch.arange(cfg.batch + 1, device=dev, dtype=torch.int32) * self.pages_per_seq
        self.kv_indices = torch.randperm(pages, generator=gen, device=dev).to(torch.int32)
        self.k_pool = _normal((pages, kvh, self.page, d), 1.0, gen, dev)      # holds the prefilled context
        self.v_pool = _normal((pages, kvh, self.page, d), 1.0, gen, dev)
        self.heads = torch.arange(kvh, device=dev)
        # the pages a decode run writes into (those that hold positions >= context), for snapshots
        first = cfg.context // self.page
        self.decode_pages = self.kv_indices.view(cfg.batch, self.pages_per_seq)[:, first:].reshape(-1).long()
        inv = 1.0 / (10000.0 ** (torch.arange(0, cfg.rotary_dim, 2, device=dev, dtype=torch.float32) / cfg.rotary_dim))
        ang = torch.arange(max_len, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()                   # [max_len, rotary_dim / 2]

    def _rope(self, x, pos):
        r = self.cfg.rotary_dim
        cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)   # [1, r/2]
        a, b = x[..., : r // 2].float(), x[..., r // 2: r].float()
        rot = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1).to(x.dtype)
        return torch.cat([rot, x[..., r:]], dim=-1)

    def __call__(self, x, pos, mask):
        cfg = self.cfg
        b, qh, kvh, d = x.shape[0], cfg.q_heads, cfg.kv_heads, cfg.head_dim
        qg = (x @ self.w_qg.t()).view(b, qh, 2, d)
        q, gate = qg[:, :, 0], qg[:, :, 1]
        kv = (x @ self.w_kv.t()).view(b, 2, kvh, d)
        k, v = kv[:, 0], kv[:, 1]
        norm = lambda t: (t.float() * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + cfg.eps)).to(t.dtype)
        q, k = self._rope(norm(q), pos), self._rope(norm(k), pos)
        # page table of the batch (every sequence has the same length here, so the CSR rows form a matrix)
        table = self.kv_indices.view(b, self.pages_per_seq).long()
        page_of_pos = table.index_select(1, pos // self.page)         # [b, 1]
        slot = (pos % self.page).view(1, 1)
        self.k_pool.index_put_((page_of_pos, self.heads.view(1, kvh), slot), k)
        self.v_pool.index_put_((page_of_pos, self.heads.view(1, kvh), slot), v)
        group = qh // kvh                                           # query heads per kv head share its K and V
        qv = q.reshape(b * kvh, group, d)
        gather = lambda pool: (pool.index_select(0, table.reshape(-1))
                               .view(b, self.pages_per_seq, kvh, self.page, d).permute(0, 2, 1, 3, 4)
                               .reshape(b * kvh, self.pages_per_seq * self.page, d))
        kc, vc = gather(self.k_pool), gather(self.v_pool)
        scores = torch.bmm(qv, kc.transpose(1, 2)).float() * (1.0 / math.sqrt(d)) + mask   # [b*kvh, group, L]
        probs = torch.softmax(scores, dim=-1).to(x.dtype)
        out = torch.bmm(probs, vc).view(b, qh, d) * torch.sigmoid(gate.float()).to(x.dtype)
        return out.reshape(b, qh * d) @ self.w_o.t()


class _GatedDeltaNet:
    """Stand-in for a GatedDeltaNet layer (torch operators): input projection, causal depth-wise
    convolution over the last `conv_kernel` tokens, gated delta-rule update of a per-head
    [head_dim, head_dim] f32 state, gated RMS norm, output projection."""

    def __init__(self, cfg: HybridConfig, gen, dev):
        h, vh, qkh, d = cfg.hidden, cfg.gdn_v_heads, cfg.gdn_qk_heads, cfg.gdn_head_dim
        self.cfg = cfg
        self.conv_channels = 2 * qkh * d + vh * d
        self.w_in = _normal((self.conv_channels + vh * d + 2 * vh, h), 0.02, gen, dev)   # q, k, v | z | b, a
        self.w_conv = _normal((self.conv_channels, cfg.conv_kernel), 0.3, gen, dev, torch.float32)
        self.w_out = _normal((h, vh * d), 0.02, gen, dev)
        self.a_log = torch.zeros(vh, device=dev)
        self.dt_bias = torch.zeros(vh, device=dev)
        self.norm_w = torch.ones(d, device=dev)
        self.conv_state = torch.zeros((cfg.batch, self.conv_channels, cfg.conv_kernel - 1), device=dev)
        self.state = _normal((cfg.batch, vh, d, d), 0.05, gen, dev, torch.float32)        # [B, heads, k, v]

    def __call__(self, x):
        cfg = self.cfg
        b, vh, qkh, d = x.shape[0], cfg.gdn_v_heads, cfg.gdn_qk_heads, cfg.gdn_head_dim
        proj = x @ self.w_in.t()
        qkv, z, ba = torch.split(proj, [self.conv_channels, vh * d, 2 * vh], dim=-1)
        window = torch.cat([self.conv_state, qkv.float().unsqueeze(-1)], dim=-1)      # [B, C, kernel]
        self.conv_state.copy_(window[..., 1:])
        qkv = torch.nn.functional.silu((window * self.w_conv).sum(-1))
        q, k, v = torch.split(qkv, [qkh * d, qkh * d, vh * d], dim=-1)
        unit = lambda t: t * torch.rsqrt(t.pow(2).sum(-1, keepdim=True) + 1e-6)
        rep = vh // qkh
        q = unit(q.view(b, qkh, d)).repeat_interleave(rep, dim=1) * (d ** -0.5)
        k = unit(k.view(b, qkh, d)).repeat_interleave(rep, dim=1)
        v = v.view(b, vh, d)
        beta = torch.sigmoid(ba[:, :vh].float())
        decay = torch.exp(-torch.exp(self.a_log) * torch.nn.functional.softplus(ba[:, vh:].float() + self.dt_bias))
        s = self.state
        s.mul_(decay[:, :, None, None])
        delta = (v - torch.einsum("bhkv,bhk->bhv", s, k)) * beta[:, :, None]
        s.add_(k.unsqueeze(-1) * delta.unsqueeze(-2))
        o = torch.einsum("bhkv,bhk->bhv", s, q)
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + cfg.eps) * self.norm_w
        o = (o * torch.nn.functional.silu(z.float().view(b, vh, d))).to(x.dtype)
        return o.reshape(b, vh * d) @ self.w_out.t()


class HybridDecoder:
    """Random-initialised model + decode state on one GPU. `step()` advances every sequence of
    the batch by one token; `capture()` records one step in a CUDA graph."""

    def __init__(self, cfg: HybridConfig, device: int = 0, keep_linear_scales: bool = False):
        self.cfg = cfg
        dev = torch.device("cuda", device)
        self.dev = dev
        self.max_len = cfg.context + cfg.new_tokens
        gen = torch.Generator(device=dev).manual_seed(cfg.seed)
        self.stream = torch.cuda.Stream(dev)     # library contexts are bound to it; graphs capture on it
        with torch.cuda.stream(self.stream):
            self.ctx = ops.Context(device)
            self.gemm = ops.GemmContext(device)
            h, b = cfg.hidden, cfg.batch
            self.embed = _normal((cfg.vocab, h), 0.02, gen, dev)
            self.lm_head = _normal((cfg.vocab, h), 0.02, gen, dev)
            self.input_norm = [torch.ones(h, dtype=torch.bfloat16, device=dev) for _ in range(cfg.layers + 1)]
            self.mixers, self.blocks = [], []
            for layer in range(cfg.layers):
                self.mixers.append(_Attention(cfg, gen, dev, self.max_len) if cfg.is_attention(layer)
                                   else _GatedDeltaNet(cfg, gen, dev))
                self.blocks.append(_MoeBlock(self.ctx, cfg, gen, dev, keep_linear_scales))
            self.plan = ops.MoePlan(self.ctx, ops.MoePlanConfig(
                max_num_tokens=b, hidden_size=h, intermediate_size=cfg.inter, num_experts=cfg.experts,
                top_k=cfg.top_k, backend=capi.MOE_BACKEND_NVFP4))
            self.ws = torch.zeros(self.plan.layer_workspace_size(b, cfg.shared_inter), dtype=torch.uint8, device=dev)
            # static buffers of a step
            self.tokens = torch.randint(0, cfg.vocab, (b,), generator=gen, device=dev)
            self.pos = torch.full((1,), cfg.context, dtype=torch.long, device=dev)
            # one entry per cache slot of a sequence's pages (the tail past max_len stays masked)
            slots = (self.max_len + cfg.page_size - 1) // cfg.page_size * cfg.page_size
            self.mask = torch.full((1, 1, slots), float("-inf"), device=dev)
            self.mask[..., : cfg.context] = 0.0
            self.x = torch.empty((b, h), dtype=torch.bfloat16, device=dev)
            self.residual = torch.empty((b, h), dtype=torch.bfloat16, device=dev)
            self.packed = torch.empty((b, h // 2), dtype=torch.uint8, device=dev)
            self.tiled = torch.zeros(ops.nvfp4_tiled_scale_bytes(b, h), dtype=torch.uint8, device=dev)
            self.logits = torch.empty((b, cfg.vocab), dtype=torch.bfloat16, device=dev)
            self.stale_mix = _normal((b, h), 0.1, gen, dev)
            self.ids = torch.empty((b, cfg.top_k), dtype=torch.int32, device=dev)
            self.weights = torch.empty((b, cfg.top_k), dtype=torch.float32, device=dev)
        self.stream.synchronize()
        self.graphs = {}
        self.trace = None    # list of per-layer dicts while a traced eager step runs
        self.position = cfg.context   # host mirror of `pos`: the cache row the next step writes

    # ---- one decode step -------------------------------------------------------------

    def step(self, mixers: bool = True):
        """One token for every sequence, enqueued on `self.stream` (must be current).
        mixers=False skips the torch stand-ins (each layer then consumes a fixed tensor in
        place of its mixer output): what remains are the calls into this library."""
        cfg, ctx = self.cfg, self.ctx
        self._advance()
        # the device-side position is clamped as well, so that no replay can index past the cache
        pos = self.pos.clamp(max=self.max_len - 1)
        self.mask.index_fill_(2, pos, 0.0)               # the new token attends to itself
        self.residual.copy_(self.embed.index_select(0, self.tokens))
        ops.rmsnorm(ctx, self.residual, self.input_norm[0], self.x, cfg.eps)
        for layer, (mixer, blk) in enumerate(zip(self.mixers, self.blocks)):
            if not mixers:
                mix = self.stale_mix.clone()
            elif cfg.is_attention(layer):
                mix = mixer(self.x, pos, self.mask)
            else:
                mix = mixer(self.x)
            # residual += mix; mix = norm(residual) (bf16) and its NVFP4 codes, one pass
            ops.fused_add_rmsnorm_nvfp4(ctx, mix, self.residual, blk.post_mixer_norm, cfg.eps, 1.0,
                                        packed=self.packed, tiled=self.tiled)
            trace_logits = None
            if self.trace is not None:
                self.trace.append(dict(normed=mix.clone(), residual_in=self.residual.clone()))
                trace_logits = torch.empty((mix.shape[0], cfg.experts), dtype=torch.float32, device=mix.device)
            # experts + shared expert + combine; residual += out; x = norm(residual) * next layer's weight
            ops.moe_layer_execute(self.plan, mix, blk.router, blk.gate_up, blk.down, self.x, self.ws,
                                  shared=blk.shared, hidden_packed=self.packed, hidden_scale_tiled=self.tiled,
                                  residual_inout=self.residual, next_norm_weight=self.input_norm[layer + 1],
                                  next_norm_eps=cfg.eps, topk_ids=self.ids, topk_weights=self.weights,
                                  router_logits=trace_logits)
            if self.trace is not None:
                self.trace[-1].update(ids=self.ids.clone(), weights=self.weights.clone(), x_out=self.x.clone(),
                                      logits=trace_logits,
                                      residual_out=self.residual.clone())
        self.gemm.gemm_bf16(self.x, self.lm_head, self.logits, alpha=1.0)
        self.tokens.copy_(self.logits.argmax(dim=-1))
        self.pos.add_(1)

    def _advance(self):
        if not torch.cuda.is_current_stream_capturing():
            if self.position >= self.max_len:
                raise RuntimeError(f"decode position {self.position} is past the cache ({self.max_len} rows)")
            self.position += 1

    def replay(self, graph):
        """Replay a captured step (keeps the host-side position in step with the device's)."""
        self._advance()
        graph.replay()

    def capture(self, mixers: bool = True):
        """Record one step in a CUDA graph (a decode step is some hundreds of short kernels:
        launched eagerly it is bound by the host)."""
        key = bool(mixers)
        if key in self.graphs:
            return self.graphs[key]
        saved = self.snapshot()
        with torch.cuda.stream(self.stream):
            self.ctx.use_current_stream()
            for _ in range(2):                      # warm-up: lazy initialisation happens outside the capture
                self.step(mixers)
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                self.step(mixers)
            self.stream.synchronize()
        self.restore(saved)
        self.graphs[key] = graph
        return graph

    # ---- decode state (for repeatable runs) ---------------------------------------------

    def _state_tensors(self):
        """(tensor, pages) of everything a step changes besides its scratch buffers; `pages` is None
        or, for a KV-cache page pool, the ids of the pages a decode run writes into."""
        out = [(self.tokens, None), (self.pos, None), (self.mask, None)]
        for m in self.mixers:
            if isinstance(m, _Attention):
                out += [(m.k_pool, m.decode_pages), (m.v_pool, m.decode_pages)]
            else:
                out += [(m.conv_state, None), (m.state, None)]
        return out

    def snapshot(self):
        """Copies of the state tensors (of a KV cache only the pages a decode run writes). Runs on
        the decode stream, which does not synchronise with the default stream."""
        snap = [self.position]
        with torch.cuda.stream(self.stream):
            for t, pages in self._state_tensors():
                snap.append(t.clone() if pages is None else t.index_select(0, pages))
        self.stream.synchronize()
        return snap

    def restore(self, snap):
        self.position = snap[0]
        with torch.cuda.stream(self.stream):
            for (t, pages), s in zip(self._state_tensors(), snap[1:]):
                if pages is None:
                    t.copy_(s)
                else:
                    t.index_copy_(0, pages, s)
        self.stream.synchronize()

    # ---- measurement ------------------------------------------------------------------------

    def time_steps(self, steps: int, mixers: bool = True, warmup: int = 3) -> float:
        """Mean ms per step over `steps` graph replays (CUDA events on the replay stream)."""
        graph = self.capture(mixers)
        saved = self.snapshot()
        steps = min(steps, self.max_len - self.position - warmup)
        if steps <= 0:
            raise RuntimeError("no room left in the cache for timed steps")
        with torch.cuda.stream(self.stream):
            for _ in range(warmup):
                self.replay(graph)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(self.stream)
            for _ in range(steps):
                self.replay(graph)
            end.record(self.stream)
            end.synchronize()
        ms = begin.elapsed_time(end) / steps
        self.restore(saved)
        return ms


def measure(steps: int | None = None, cfg: HybridConfig | None = None) -> dict:
    """Build the decoder, time `steps` decoded tokens per sequence (default: the configuration's 256)
    as CUDA-graph replays with and without the mixers, and return the record `main` prints."""
    cfg = cfg or HybridConfig()
    steps = cfg.new_tokens if steps is None else steps
    model = HybridDecoder(cfg)
    timed = min(steps, model.max_len - model.position - 3)
    full = model.time_steps(steps, mixers=True)
    lib = model.time_steps(steps, mixers=False)
    err = model.ctx.read_device_error()
    moe_bytes = cfg.moe_weight_bytes_per_layer() * cfg.layers
    return {
        "metric": "hybrid decode tokens/s (batch x steps / time), CUDA graph replay", "value": cfg.batch / (full * 1e-3),
        "unit": "tokens/s", "ms_per_step": full, "library_ms_per_step": lib, "library_share": lib / full,
        "library_calls": "rmsnorm, fused add+rmsnorm+NVFP4, MoE layer (+ residual add + next norm), LM head",
        "moe_weight_bytes_per_step": moe_bytes, "moe_weight_stream_gbs": moe_bytes / (lib * 1e-3) / 1e9,
        "mixers": f"torch stand-ins (gated attention over a paged KV cache, {cfg.page_size}-token pages behind a CSR "
                  "page table; GatedDeltaNet recurrence)",
        "config": {k: getattr(cfg, k) for k in ("layers", "hidden", "experts", "top_k", "inter", "shared_inter",
                                                 "batch", "context", "vocab", "page_size")},
        "steps": timed, "device_error": err, "data": "synthetic"}


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--steps", type=int, default=HybridConfig.new_tokens)
    ap.add_argument("--layers", type=int, default=HybridConfig.layers)
    ap.add_argument("--batch", type=int, default=HybridConfig.batch)
    ap.add_argument("--context", type=int, default=HybridConfig.context)
    args = ap.parse_args()
    cfg = HybridConfig(layers=args.layers, batch=args.batch, context=args.context)
    print(json.dumps(measure(args.steps, cfg)))


if __name__ == "__main__":
    main()
