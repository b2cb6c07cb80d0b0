"""Synthetic MoE-layer workloads with the shapes and value distributions of the
benchmark configurations, generated on the device from a seed.

The reference publishes no dataset for this path; the configurations name only
shapes and distributions (activations ~ N(0, 1), weights ~ N(0, 0.02), a Zipf-like
additive router bias), so seeded synthetic tensors stand in for real checkpoints.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import capi, ops


@dataclass
class LayerConfig:
    name: str
    tokens: int
    hidden: int
    experts: int
    top_k: int
    inter: int
    shared_inter: int = 0
    nvfp4: bool = True
    zipf_s: float = 0.0
    fp8: bool = False   # e4m3 experts with 128 x 128 block scales (nvfp4 must then be False)

    @property
    def dtype_name(self) -> str:
        return "nvfp4" if self.nvfp4 else "fp8" if self.fp8 else "bf16"


# Qwen3-Next-shaped prefill layer: 8192 tokens, 512 experts, top-10 + shared expert, NVFP4
PREFILL_NVFP4 = LayerConfig("qwen3next_moe_prefill_nvfp4", 8192, 2048, 512, 10, 512, 512, True, 1.1)
# per-rank slice of the expert-parallel configuration (4096 tokens per rank)
EP_NVFP4 = LayerConfig("qwen3next_moe_ep_nvfp4", 4096, 2048, 512, 10, 512, 512, True, 1.1)
TINY_BF16 = LayerConfig("tiny_bf16", 16, 256, 8, 2, 128, 0, False, 0.0)
# decode batch of the same layer as the prefill workload (what one layer of the 48-layer hybrid decode
# sees: 128 sequences, unbiased router, so almost every expert is hit by a few rows)
DECODE_NVFP4 = LayerConfig("qwen3next_moe_decode_nvfp4", 128, 2048, 512, 10, 512, 512, True, 0.0)
# Qwen3-30B-A3B-shaped decode batch: 64 tokens, 128 experts, top-8, FP8 block-scaled, no shared expert
DECODE_FP8 = LayerConfig("qwen3_30b_a3b_moe_decode_fp8", 64, 2048, 128, 8, 768, 0, False, 0.0, True)


def _normal_bf16(shape, std, gen, device, chunk_rows=64):
    """N(0, std) in bf16, generated in slices of the leading dimension to bound f32 scratch."""
    out = torch.empty(shape, dtype=torch.bfloat16, device=device)
    lead = shape[0]
    for s in range(0, lead, chunk_rows):
        e = min(lead, s + chunk_rows)
        out[s:e] = (torch.randn((e - s, *shape[1:]), generator=gen, device=device, dtype=torch.float32)
                    * std).to(torch.bfloat16)
    return out


class LayerData:
    """Weights (quantised once, like a weight loader would) and inputs of one layer.

    ``expert_range`` = (first, count) keeps only that slice of the routed experts on
    this device (expert parallelism); router and shared expert are always whole.
    ``placement`` (optional, a permutation of the expert ids) stores logical expert
    ``placement[p]`` at physical position ``p``: router rows, router bias and expert
    weights are laid out in physical order, so every id the layer reports is a physical
    one and ``expert_range`` slices physical positions. This is how a weight loader
    spreads hot experts over ranks. ``balance_world`` = n > 1 derives the placement here:
    the router is run on a seeded calibration batch (the same on every rank, plain tensor
    ops at set-up time) and ``ep.balanced_placement`` evens the per-rank route counts.
    ``hot_experts`` = H > 0 (with ``balance_world``) additionally REPLICATES the H experts
    that got the most routes on the calibration batch: every rank keeps a copy of them
    after its own experts (``hot_positions`` lists their physical positions, the same on
    every rank), so a token's routes to a hot expert are served where the token lives and
    neither the token nor a partial sum crosses NVLink for them. ``slot_id_map`` turns the
    router's ids into the expert slots of this layout.
    """

    def __init__(self, cfg: LayerConfig, ctx: ops.Context, seed: int = 0, expert_range=None,
                 token_seed: int | None = None, keep_bf16: bool = False, placement=None,
                 balance_world: int = 0, calibration_tokens: int = 8192, hot_experts: int = 0,
                 hot_positions=None):
        dev = torch.device("cuda", ctx.device)
        self.cfg = cfg
        first, count = expert_range if expert_range is not None else (0, cfg.experts)
        self.expert_range = (first, count)
        gw = torch.Generator(device=dev)
        gw.manual_seed(1000 * seed + 1)
        h, i, s = cfg.hidden, cfg.inter, cfg.shared_inter
        self.router = _normal_bf16((cfg.experts, h), 0.02, gw, dev)
        self.bias = None
        if cfg.zipf_s > 0:
            perm = torch.randperm(cfg.experts, generator=gw, device=dev)
            self.bias = (-cfg.zipf_s * torch.log1p(perm.to(torch.float32))).contiguous()
        logical = list(range(cfg.experts))
        if placement is None and balance_world > 1:
            from .ep import balanced_placement
            gc = torch.Generator(device=dev)
            gc.manual_seed(1000 * seed + 999)
            x = _normal_bf16((calibration_tokens, h), 1.0, gc, dev, chunk_rows=1024)
            logits = x.float() @ self.router.float().t()
            if self.bias is not None:
                logits += self.bias
            ids = logits.topk(cfg.top_k, dim=1).indices
            counts = torch.bincount(ids.flatten(), minlength=cfg.experts).cpu().tolist()
            hot_logical = []
            if hot_experts > 0:
                from .ep import hottest_experts
                hot_logical = hottest_experts(counts, hot_experts)
                counts = [0 if e in set(hot_logical) else c for e, c in enumerate(counts)]
            placement = balanced_placement(counts, balance_world)
            if hot_logical:
                where = {e: p for p, e in enumerate(placement)}
                hot_positions = [where[e] for e in hot_logical]
            del x, logits, ids
        if placement is not None:
            logical = [int(e) for e in placement]
            if sorted(logical) != list(range(cfg.experts)):
                raise ValueError("placement must be a permutation of the expert ids")
            index = torch.tensor(logical, dtype=torch.long, device=dev)
            self.router = self.router.index_select(0, index).contiguous()
            if self.bias is not None:
                self.bias = self.bias.index_select(0, index).contiguous()
        self.placement = logical
        self.hot_positions = [int(p) for p in hot_positions] if hot_positions else []
        # routed experts: every expert is generated from its own seed so that all ranks agree; this rank
        # keeps its slice of the physical positions, followed by its replicas of the hot experts
        local = list(range(first, first + count)) + (self.hot_positions if expert_range is not None else [])
        self.local_positions = local
        gate_up = torch.empty((len(local), 2 * i, h), dtype=torch.bfloat16, device=dev)
        down = torch.empty((len(local), h, i), dtype=torch.bfloat16, device=dev)
        for slot, pos in enumerate(local):
            ge = torch.Generator(device=dev)
            ge.manual_seed(1000 * seed + 100 + logical[pos])
            gate_up[slot] = (torch.randn((2 * i, h), generator=ge, device=dev) * 0.02).to(torch.bfloat16)
            down[slot] = (torch.randn((h, i), generator=ge, device=dev) * 0.02).to(torch.bfloat16)
        self.shared = None
        if s:
            sgu = _normal_bf16((1, 2 * s, h), 0.02, gw, dev)
            sdn = _normal_bf16((1, h, s), 0.02, gw, dev)
            sgate = _normal_bf16((1, h), 0.02, gw, dev)
        if cfg.nvfp4:
            self.gate_up = ops.nvfp4_quantize_weight(ctx, gate_up, True)
            self.down = ops.nvfp4_quantize_weight(ctx, down, False)
            if s:
                self.shared = ops.SharedExpert(ops.nvfp4_quantize_weight(ctx, sgu, True),
                                               ops.nvfp4_quantize_weight(ctx, sdn, False), sgate, s)
            torch.cuda.synchronize(dev)
        elif cfg.fp8:
            if s:
                raise ValueError("the FP8 layer takes no shared expert")
            self.gate_up = ops.fp8_quantize_weight(ctx, gate_up)
            self.down = ops.fp8_quantize_weight(ctx, down)
            torch.cuda.synchronize(dev)
        else:
            self.gate_up, self.down = gate_up, down
            if s:
                self.shared = ops.SharedExpert(sgu, sdn, sgate, s)
        if keep_bf16:
            self.gate_up_bf16, self.down_bf16 = gate_up, down
            if s:
                self.shared_bf16 = (sgu, sdn, sgate)
        gt = torch.Generator(device=dev)
        gt.manual_seed(1000 * seed + 7 + (token_seed or 0))
        self.hidden = _normal_bf16((cfg.tokens, h), 1.0, gt, dev, chunk_rows=1024)

    def slot_id_map(self, rank: int, world: int):
        """i32 [experts]: the expert SLOT (rank * slots_per_rank + index on that rank) a route of a
        token that lives on ``rank`` goes to, per physical expert id: the owner's slot for an ordinary
        expert, this rank's own replica for a hot one. None without replicated experts."""
        if not self.hot_positions:
            return None
        from .ep import slot_id_table
        table = slot_id_table(self.cfg.experts, world, self.hot_positions, rank)
        return torch.tensor(table, dtype=torch.int32, device=self.hidden.device)

    def plan(self, ctx: ops.Context, max_tokens: int | None = None) -> ops.MoePlan:
        cfg = self.cfg
        first, count = self.expert_range
        return ops.MoePlan(ctx, ops.MoePlanConfig(
            max_num_tokens=max_tokens or cfg.tokens, hidden_size=cfg.hidden, intermediate_size=cfg.inter,
            num_experts=cfg.experts, top_k=cfg.top_k, local_expert_offset=first, local_num_experts=count,
            backend=capi.MOE_BACKEND_NVFP4 if cfg.nvfp4
            else capi.MOE_BACKEND_FP8_BLOCKSCALE if cfg.fp8 else capi.MOE_BACKEND_STAGED_BF16,
            route_mode=capi.MOE_ROUTE_ROUTER_LOGITS))

    def weight_bytes_per_expert(self):
        """(gate_up bytes, down bytes) of one routed expert as the kernels read them."""
        cfg = self.cfg
        if cfg.nvfp4:
            return (2 * cfg.inter * cfg.hidden // 2 + 2 * cfg.inter * cfg.hidden // 16,
                    cfg.hidden * cfg.inter // 2 + cfg.hidden * cfg.inter // 16)
        if cfg.fp8:
            blocks = (2 * cfg.inter // 128) * (cfg.hidden // 128)
            return 2 * cfg.inter * cfg.hidden + 4 * blocks, cfg.hidden * cfg.inter + 2 * blocks
        return 2 * cfg.inter * cfg.hidden * 2, cfg.hidden * cfg.inter * 2
