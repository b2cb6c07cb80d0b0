#!/usr/bin/env python3
"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the whole MoE layer (router logits -> top-k -> permute ->
grouped gate_up GEMM + SwiGLU -> grouped down GEMM -> shared expert -> combine) over
one batch of synthetic tokens. At N = 1 the workload is the NVFP4 prefill layer
(8192 tokens, hidden 2048, 512 experts, top-10 + shared expert, Zipf-skewed router);
at N > 1 it is the expert-parallel variant with 4096 tokens per rank (weak scaling),
launched one process per GPU by torch.distributed.run. `--workload decode_fp8` (N = 1)
times the FP8 block-scaled decode batch instead (64 tokens, 128 experts, top-8) and
`--workload decode_nvfp4` a 128-token decode batch of the NVFP4 layer (unbiased router).

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events, max over
ranks) with inputs resident in HBM; `e2e` goes through the same C-ABI call with the
tokens starting in pinned host memory and the result read back to the host inside
the timed region. Timing: blocks of exactly `--steps` steps run back to back for at
least half a second of GPU time, every block bracketed by CUDA events; `ms_per_step`
is the median block divided by `--steps` (p10 / p90 beside it), so the figure is taken
at the clocks the GPU sustains, not in a cold 10 ms burst. `roofline` describes the
dominant kernel (grouped gate_up GEMM), timed with CUDA events around that kernel, against
the resource that binds that launch; `stages` gives the HBM fractions of the routing,
permute and combine kernels; `parity` is a sampled check of the timed layer's results
against the CPU oracle (expert ids and permutation of all tokens bit for bit, outputs of a
sample of tokens within tolerance), run once after the timed loops; `cpu_baseline`
times the CPU oracle on a bounded sample of the same workload on this machine's host
cores; `secondary` (N = 1) holds the decode workloads measured after the headline: the two decode
batches of one layer and the 48-layer hybrid decode loop (`qs3_b200/hybrid_decode.py`).

`--impl reference` times the CPU oracle alone (the reference has no CPU MoE path of
its own and its GPU path has no NVFP4 kernels, so the restated algorithm is the only
reference implementation of this workload that exists). That arm generates and
quantises its inputs on the host and loads nothing of the product library.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _quantiles(xs):
    xs = sorted(xs)
    pick = lambda q: xs[min(len(xs) - 1, max(0, int(round(q * (len(xs) - 1)))))]
    return statistics.median(xs), pick(0.1), pick(0.9)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(names, s[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------ CPU oracle leg ---

def _host_layer(cfg, seed, sample_tokens):
    """Inputs of the layer generated and quantised on the host with numpy and the oracle's own
    quantisers (same shapes and distributions as ``qs3_b200.workload.LayerData``: activations
    N(0,1), weights N(0,0.02), Zipf-like router bias), for the reference arm, which must not
    touch the product library. Only the first ``sample_tokens`` tokens are generated, and only
    the experts those tokens are routed to get weights (the others are never read)."""
    import numpy as np
    from oracle import binding as orc
    rng = np.random.default_rng([seed, 1])
    h, i, s, e = cfg.hidden, cfg.inter, cfg.shared_inter, cfg.experts
    bf = lambda a: orc.f32_to_bf16(np.asarray(a, dtype=np.float32))
    host = {"router": bf(rng.standard_normal((e, h), dtype=np.float32) * 0.02), "bias": None, "shared": None}
    if cfg.zipf_s > 0:
        host["bias"] = (-cfg.zipf_s * np.log1p(rng.permutation(e).astype(np.float64))).astype(np.float32)
    host["hidden"] = bf(np.random.default_rng([seed, 7]).standard_normal((sample_tokens, h), dtype=np.float32))
    logits = orc.gemm_bf16(host["hidden"], host["router"], "f32")
    ids, _ = orc.router_topk(logits, cfg.top_k, 0, True, 1.0, host["bias"])
    hit = np.unique(ids)
    if cfg.nvfp4:
        gu = [np.zeros((e, 2 * i, h // 2), np.uint8), np.zeros((e, 2 * i, h // 16), np.uint8), np.ones(e, np.float32)]
        dn = [np.zeros((e, h, i // 2), np.uint8), np.zeros((e, h, i // 16), np.uint8), np.ones(e, np.float32)]
    else:
        gu = [np.zeros((e, 2 * i, h), np.uint8), np.ones((e, 2 * i // 128, h // 128), np.float32)]
        dn = [np.zeros((e, h, i), np.uint8), np.ones((e, h // 128, (i + 127) // 128), np.float32)]
    for x in hit:
        ge = np.random.default_rng([seed, 100 + int(x)])
        w1 = bf(ge.standard_normal((1, 2 * i, h), dtype=np.float32) * 0.02)
        w2 = bf(ge.standard_normal((1, h, i), dtype=np.float32) * 0.02)
        if cfg.nvfp4:
            p, l, _t, g = orc.nvfp4_quantize_weight(w1, False, tiled=False)
            gu[0][x], gu[1][x], gu[2][x] = p[0], l[0], g[0]
            p, l, _t, g = orc.nvfp4_quantize_weight(w2, False, tiled=False)
            dn[0][x], dn[1][x], dn[2][x] = p[0], l[0], g[0]
        else:
            c, sc = orc.fp8_quantize_weight(w1)
            gu[0][x], gu[1][x] = c[0], sc[0]
            c, sc = orc.fp8_quantize_weight(w2)
            dn[0][x], dn[1][x] = c[0], sc[0]
    host["gu"], host["d"] = tuple(gu), tuple(dn)
    if s:
        q = lambda w: (lambda r: (r[0], r[1], r[3]))(orc.nvfp4_quantize_weight(w, False, tiled=False))
        host["shared"] = dict(gu=q(bf(rng.standard_normal((1, 2 * s, h), dtype=np.float32) * 0.02)),
                              d=q(bf(rng.standard_normal((1, h, s), dtype=np.float32) * 0.02)),
                              gate_w=bf(rng.standard_normal((1, h), dtype=np.float32) * 0.02))
    return host, int(hit.size)


def time_oracle(host, cfg, target_seconds=20.0, max_tokens=4096):
    """tokens/s of the CPU oracle on a bounded sample sized for roughly target_seconds / 2 or more
    of work: a prefix of the batch, or the whole batch several times when it is small. Uses
    every core this process may run on, whatever OMP_NUM_THREADS the launcher exported."""
    import numpy as np
    from oracle import binding as orc
    from oracle import parity
    orc.build()
    orc.set_num_threads()
    avail = min(cfg.tokens, host["hidden"].shape[0])
    probe = np.arange(min(8, avail))
    parity.oracle_layer(host, cfg, probe)          # warm the thread pool and the caches
    t0 = time.perf_counter()
    parity.oracle_layer(host, cfg, probe)
    per_token = (time.perf_counter() - t0) / len(probe)
    n = int(max(8, min(max_tokens, avail, target_seconds / max(per_token, 1e-6))))
    sample = np.arange(n)
    reps, done, t0 = 0, 0.0, time.perf_counter()
    while True:
        parity.oracle_layer(host, cfg, sample)
        reps += 1
        done = time.perf_counter() - t0
        if n < cfg.tokens or done >= 0.5 * target_seconds or reps >= 200:
            break
    return n * reps / done, n * reps, done, orc.num_threads()


# ----------------------------------------------------------------------- main legs ---

def _workload(args, module=None):
    """The layer configuration the flags select: at N = 1 the NVFP4 prefill layer unless
    --workload names a decode batch; at N > 1 the expert-parallel NVFP4 layer."""
    if module is None:
        from qs3_b200 import workload as module
    if args.gpus == 1:
        return {"decode_fp8": module.DECODE_FP8, "decode_nvfp4": module.DECODE_NVFP4}.get(
            args.workload, module.PREFILL_NVFP4)
    if args.workload != "prefill_nvfp4":
        raise SystemExit("only the NVFP4 layer runs expert-parallel")
    return module.EP_NVFP4


def _config(cfg, world, placement="balanced", hot=0):
    """The `config` object of the JSON line, identical for both arms."""
    weights_gb = cfg.experts * 3 * cfg.inter * cfg.hidden * (0.5625 if cfg.nvfp4 else 1.0 if cfg.fp8 else 2.0) / 1e9
    return {"workload": cfg.name, "tokens_per_gpu": cfg.tokens, "hidden": cfg.hidden, "experts": cfg.experts,
            "top_k": cfg.top_k, "intermediate": cfg.inter, "shared_intermediate": cfg.shared_inter,
            "router_bias": f"zipf(s={cfg.zipf_s})", "parallelism": "single" if world == 1 else f"ep{world}",
            "expert_placement": "all local" if world == 1 else
            ("contiguous blocks of expert ids" if placement == "contiguous" else
             "even counts per rank, load-balanced on a calibration batch (longest-processing-time rule)"
             + (f"; the {hot} hottest experts of that batch are also replicated on every rank, so their routes "
                "are served where the token lives" if hot else "")),
            "l2_policy": f"inputs_exceed_l2 (expert weights ~{weights_gb:.1f} GB per pass)"}


class _RefConfigs:
    """The benchmark layer shapes for the reference arm, which imports neither torch nor the
    product package (``qs3_b200.workload`` pulls both in). Kept equal to the constants there;
    ``tests/test_abi_host.py`` compares the two."""

    @staticmethod
    def make():
        from types import SimpleNamespace as NS

        def cfg(name, tokens, hidden, experts, top_k, inter, shared, nvfp4, zipf, fp8=False):
            return NS(name=name, tokens=tokens, hidden=hidden, experts=experts, top_k=top_k, inter=inter,
                      shared_inter=shared, nvfp4=nvfp4, zipf_s=zipf, fp8=fp8,
                      dtype_name="nvfp4" if nvfp4 else "fp8" if fp8 else "bf16")
        return NS(PREFILL_NVFP4=cfg("qwen3next_moe_prefill_nvfp4", 8192, 2048, 512, 10, 512, 512, True, 1.1),
                  EP_NVFP4=cfg("qwen3next_moe_ep_nvfp4", 4096, 2048, 512, 10, 512, 512, True, 1.1),
                  DECODE_NVFP4=cfg("qwen3next_moe_decode_nvfp4", 128, 2048, 512, 10, 512, 512, True, 0.0),
                  DECODE_FP8=cfg("qwen3_30b_a3b_moe_decode_fp8", 64, 2048, 128, 8, 768, 0, False, 0.0, True))


def run_reference(args, rank, world):
    """Reference arm: the CPU restatement on the host cores, rank 0 only. Inputs are generated
    and quantised on the host; neither torch nor the product library is loaded."""
    if rank != 0:
        return
    cfg = _workload(args, _RefConfigs.make())
    from oracle import binding as orc
    orc.build()
    cores = orc.set_num_threads()
    per_step = max(2.0, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    sample_tokens = min(cfg.tokens, 4096)
    host, hit = _host_layer(cfg, 0, sample_tokens)
    vals = []
    n = dt = 0
    for step in range(args.warmup + args.steps):
        v, n, dt, cores = time_oracle(host, cfg, target_seconds=per_step, max_tokens=sample_tokens)
        if step >= args.warmup:
            vals.append(v)
    value = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * dt, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": cfg.dtype_name, "data": "synthetic",
        "config": _config(cfg, args.gpus, args.placement, 0 if args.gpus == 1 else args.hot_experts),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{n} tokens per step (a prefix of the batch, or the batch repeated), whole layer "
                                   f"on the CPU oracle; inputs generated on the host, {hit} experts hit"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def timed_blocks(step, steps, barrier, all_max, min_seconds, clock_index=None, max_blocks=500):
    """Run blocks of ``steps`` calls of ``step`` back to back for at least ``min_seconds`` of GPU
    time, each block bracketed by CUDA events. Returns (per-block ms list, element-wise max over
    ranks; total ms first to last event; clock summary)."""
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for _ in range(steps):
        step()
    b.record()
    barrier()
    one = all_max([a.elapsed_time(b)])[0]
    blocks = int(max(5, min(max_blocks, min_seconds * 1000.0 / max(one, 1e-3) + 1)))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    sampler = ClockSampler(clock_index) if clock_index is not None else None
    if sampler is not None:
        sampler.__enter__()
    barrier()
    torch.cuda.cudart().cudaProfilerStart()  # lets `ncu --profile-from-start off` see only this region
    ev[0].record()
    for blk in range(blocks):
        for _ in range(steps):
            step()
        ev[blk + 1].record()
    barrier()
    torch.cuda.cudart().cudaProfilerStop()
    if sampler is not None:
        sampler.__exit__(None, None, None)
    per_block = all_max([ev[i].elapsed_time(ev[i + 1]) for i in range(blocks)])
    total = all_max([ev[0].elapsed_time(ev[blocks])])[0]
    return per_block, total, (sampler.summary() if sampler is not None else None)


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from qs3_b200 import ops, workload

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    ctx = ops.Context(local_rank)
    ctx.validate_target()

    if world == 1:
        cfg = _workload(args)
        if args.tokens or args.experts:
            # reduced case for profiler captures only (never a reported bench value)
            import dataclasses
            cfg = dataclasses.replace(cfg, name=cfg.name + "_reduced", tokens=args.tokens or cfg.tokens,
                                      experts=args.experts or cfg.experts)
        data = workload.LayerData(cfg, ctx, seed=0)
        layer = SingleGpuLayer(ctx, data)
        if not args.no_graph and not args.kernels_only:  # profiler captures see plain launches
            layer.try_capture()
    else:
        from qs3_b200 import ep
        cfg = workload.EP_NVFP4
        per = cfg.experts // world
        data = workload.LayerData(cfg, ctx, seed=0, expert_range=(rank * per, per), token_seed=rank + 1,
                                  balance_world=0 if args.placement == "contiguous" else world,
                                  hot_experts=0 if args.placement == "contiguous" else args.hot_experts)
        layer = ep.ExpertParallelLayer(ctx, data, rank, world)
        if not args.no_graph and not args.kernels_only:
            layer.try_capture()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def all_max(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # ---- value: inputs resident in HBM ----
    for _ in range(args.warmup):
        layer.step()
    barrier()
    launches0 = ops.launch_count()
    min_s = 0.02 if args.kernels_only else args.min_seconds
    blocks_ms, total_ms, clocks = timed_blocks(layer.step, args.steps, barrier, all_max, min_s, local_rank)
    launches = ops.launch_count() - launches0
    if ctx.read_device_error() != 0:
        raise RuntimeError("a tensor-core kernel reported a bounded-wait expiry")
    block_med, block_p10, block_p90 = _quantiles(blocks_ms)

    # ---- e2e: tokens start in pinned host memory, result is read back ----
    h_in = torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16).pin_memory()
    h_in.copy_(data.hidden.cpu())
    h_out = torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16).pin_memory()
    e2e_med = float("nan")
    e2e_blocks = 0
    if not args.kernels_only:
        pipe = E2EPipeline(layer, cfg, dev)
        pipe.run(min(3, max(2, args.warmup)), h_in, h_out)
        e_ms, _tot, _ = timed_blocks(lambda: pipe.run(args.steps, h_in, h_out), 1, barrier, all_max,
                                     0.6 * args.min_seconds, max_blocks=100)
        e2e_med = _quantiles(e_ms)[0]
        e2e_blocks = len(e_ms)

    # ---- per-stage profile (separate pass, CUDA events around every stage) ----
    stage_ms = {}
    if hasattr(layer, "profile") and not args.kernels_only:
        stage_ms = layer.profile(max(3, min(args.steps, 10)))

    # ---- parity of what was timed, against the CPU oracle (after the timing) ----
    parity = None
    extra = {}
    if world == 1:
        if not args.kernels_only and not args.no_parity:
            parity = layer.parity(sample=64)
    elif not args.kernels_only:
        # every rank also holds ALL experts (same placement) for two purposes: the oracle needs the
        # weights of whatever experts a sampled token is routed to, and the weak-scaling base is the
        # single-GPU layer on one rank's 4096 tokens, timed here in the same run
        full = workload.LayerData(cfg, ctx, seed=0, token_seed=rank + 1, placement=data.placement)
        if not args.no_parity:
            parity = ep_parity(layer, full, sample=24)
            flags = all_max([0.0 if parity["ok"] else 1.0, parity["rel_l2"], float(parity["ids_mismatches"])])
            parity = dict(parity, ok_all_ranks=flags[0] == 0.0, rel_l2_max_over_ranks=flags[1],
                          ids_mismatches_max_over_ranks=int(flags[2]))
        single = SingleGpuLayer(ctx, full)
        single.try_capture()
        for _ in range(3):
            single.step()
        base_blocks, _t, _ = timed_blocks(single.step, args.steps, barrier, all_max, 0.3 * args.min_seconds)
        base_ms = _quantiles(base_blocks)[0] / args.steps
        extra["weak_base_ms"] = base_ms
        extra["efficiency_same_tokens"] = base_ms / (block_med / args.steps)
        extra["efficiency_note"] = ("weak_base_ms = the single-GPU layer (all 512 experts local) on one rank's "
                                    "4096 tokens, max over ranks, same run; efficiency_same_tokens = weak_base_ms / "
                                    "ms_per_step")
        extra["stage_ms_note"] = ("phases of a serialised pass of eager launches on rank 0 (ranks aligned by a "
                                  "barrier before each pass): they include the host's launch gaps, which the "
                                  "timed steps, replayed from a CUDA graph, do not have; 'experts/...' are the "
                                  "library's own stage events inside the experts phase")
        del single, full

    total_tokens = cfg.tokens * world
    value = total_tokens * args.steps / (block_med / 1000.0)
    e2e_value = total_tokens * args.steps / (e2e_med / 1000.0)

    hbm_gbs, peak_kind = _peaks()
    roof = layer.roofline(stage_ms, hbm_gbs, peak_kind)   # on every rank: it may run collectives at N > 1
    if rank != 0:
        return
    graphed = getattr(layer, "graph", None) is not None
    line = {
        "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": block_med / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cfg.dtype_name,
        "data": "synthetic",
        "config": _config(cfg, world, args.placement, 0 if world == 1 else args.hot_experts),
        "timing": {"blocks": len(blocks_ms), "steps_per_block": args.steps, "block_ms_median": block_med,
                   "block_ms_p10": block_p10, "block_ms_p90": block_p90, "timed_region_ms": total_ms,
                   "ms_per_step_p10": block_p10 / args.steps, "ms_per_step_p90": block_p90 / args.steps,
                   "note": "value and ms_per_step come from the median block of `steps` steps; all blocks run "
                           "back to back between one pair of barriers"},
        "e2e": {"value": e2e_value, "unit": "tokens/s",
                "h2d_bytes_per_step": h_in.numel() * 2 * world, "d2h_bytes_per_step": h_out.numel() * 2 * world,
                "blocks": e2e_blocks},
        "gpu_launches": launches if graphed is False else len(blocks_ms) * args.steps * layer.launches_per_step,
        "gpu_launches_per_step": (launches // max(1, len(blocks_ms) * args.steps)) if graphed is False
        else layer.launches_per_step,
        "cuda_graph": graphed,
        "clocks": clocks,
        "stage_ms": stage_ms,
    }
    line.update(extra)
    line["roofline"] = roof
    if hasattr(layer, "stage_rooflines"):
        line["stages"] = layer.stage_rooflines(stage_ms, hbm_gbs)
    if parity is not None:
        line["parity"] = parity
    if world == 1 and not args.no_cpu_baseline and not args.kernels_only:
        from oracle import parity as orc_parity
        host = orc_parity.host_copies(data)
        v, n, dt, cores = time_oracle(host, cfg)
        line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                                "sample": f"{n} tokens (a prefix of the batch, or the batch repeated), whole layer on the CPU oracle, {dt:.1f} s"}
        del host
    if world == 1 and args.workload == "prefill_nvfp4" and not (args.no_secondary or args.kernels_only
                                                                 or args.tokens or args.experts):
        del layer, data
        torch.cuda.empty_cache()
        line["secondary"] = secondary_workloads(ctx, args, hbm_gbs, peak_kind)
    print(json.dumps(line), flush=True)


def ep_parity(layer, full, sample):
    """Sampled check of one expert-parallel step on this rank's tokens against the CPU oracle;
    `full` holds all experts in the layer's placement (the oracle needs every expert a sampled
    token is routed to). Also checks the rank's route sort over everything it received."""
    import torch
    from oracle import binding as orc
    from oracle import parity
    cfg = layer.cfg
    out = layer.step()
    torch.cuda.synchronize()
    b = layer.backend
    host = parity.host_copies(full)
    res = parity.check_layer(host, cfg, logits=b.logits.cpu().numpy(), ids=b.ids.cpu().numpy(),
                             weights=b.wts.cpu().numpy(), out=out.cpu().view(torch.uint16).numpy(),
                             sample=sample, seed=layer.rank)
    if hasattr(layer, "routing_snapshot"):
        ids_in, wts_in, first, count, tables = layer.routing_snapshot()
        c_ref, p_ref, rr_ref, rt_ref, _ = orc.route_sort(ids_in, wts_in, first, count)
        n_rows = int(p_ref[-1])
        res["tables_exact"] = bool(np_equal(tables[0], c_ref) and np_equal(tables[1], p_ref)
                                   and np_equal(tables[2], rr_ref) and np_equal(tables[3][:n_rows], rt_ref))
        res["local_routes"] = n_rows
        res["ok"] = bool(res["ok"] and res["tables_exact"])
    return res


def np_equal(a, b):
    import numpy as np
    return bool(np.array_equal(np.asarray(a), np.asarray(b)))


def secondary_workloads(ctx, args, hbm_gbs, peak_kind):
    """The decode batches, measured after the headline so that their figures travel in the same
    record: the FP8 block-scaled decode batch (64 tokens, 128 experts, top-8) and a 128-token
    decode batch of the NVFP4 layer. Same timing method; each with its own sampled parity."""
    import torch
    from qs3_b200 import workload
    out = {}
    sync = lambda: torch.cuda.synchronize()
    same = lambda v: list(v)
    for key, cfg in (("decode_fp8", workload.DECODE_FP8), ("decode_nvfp4", workload.DECODE_NVFP4)):
        try:
            data = workload.LayerData(cfg, ctx, seed=0)
            layer = SingleGpuLayer(ctx, data)
            layer.try_capture()
            for _ in range(max(3, args.warmup)):
                layer.step()
            blocks, _total, _ = timed_blocks(layer.step, args.steps, sync, same, 0.3 * args.min_seconds)
            med = _quantiles(blocks)[0] / args.steps
            stage_ms = layer.profile(5)
            roof = layer.roofline(stage_ms, hbm_gbs, peak_kind, probe=False)
            res = {"workload": cfg.name, "ms_per_step": med, "tokens_per_s": cfg.tokens / (med * 1e-3),
                   "cuda_graph": layer.graph is not None, "stage_ms": stage_ms}
            if roof:
                res["gate_up_gemm"] = {"kernel": roof["kernel"], "ms": roof["kernel_ms"],
                                       "hbm_gbs": roof["hbm_gbs"], "frac_hbm": roof["hbm_frac"]}
                if "down_gemm" in roof:
                    res["down_gemm"] = {"ms": roof["down_gemm"]["kernel_ms"], "hbm_gbs": roof["down_gemm"]["achieved"],
                                        "frac_hbm": roof["down_gemm"]["frac"]}
            if not args.no_parity:
                p = layer.parity(sample=32)
                res["parity"] = {k: p[k] for k in ("ok", "ids_exact", "tables_exact", "rel_l2", "tokens_checked")}
            out[key] = res
            del layer, data
            torch.cuda.empty_cache()
        except Exception as exc:  # a secondary figure must not take the headline line with it
            out[key] = {"error": f"{type(exc).__name__}: {exc}"}
    if not args.no_hybrid:
        out["hybrid_decode"] = hybrid_decode_record()
    return out


def hybrid_decode_record():
    """The 48-layer hybrid decode loop around this library's MoE layer (batch 128, 4096-token context
    in a paged KV cache, 256 generated tokens per sequence, 512 experts top-10 + shared expert, NVFP4):
    tokens/s of the whole step and the share of it spent in this library's calls. The token mixers
    are torch stand-ins, so the step time is not a model-speed claim; `library_ms_per_step` is."""
    import torch
    try:
        from qs3_b200 import hybrid_decode
        t0 = time.time()
        rec = hybrid_decode.measure()
        rec["wall_s"] = round(time.time() - t0, 1)
        torch.cuda.empty_cache()
        return rec
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


class E2EPipeline:
    """End-to-end steps with host buffers: every step copies its tokens from pinned host
    memory, runs the layer through the C ABI and copies the bf16 result back to the host.
    Copies run on their own streams with two device buffers each way, so the upload of
    step i+1 and the download of step i-1 overlap the compute of step i, as a serving
    loop would do; every step's copies are inside the timed region."""

    def __init__(self, layer, cfg, dev):
        import torch
        self.torch, self.layer = torch, layer
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        mk = lambda: torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16, device=dev)
        self.x, self.y = [mk(), mk()], [mk(), mk()]
        ev = lambda: [torch.cuda.Event(), torch.cuda.Event()]
        self.in_ready, self.compute_done, self.out_copied = ev(), ev(), ev()

    def run(self, steps, h_in, h_out):
        torch = self.torch
        main = torch.cuda.current_stream()
        for i in range(steps):
            b = i & 1
            if i >= 2:
                self.h2d.wait_event(self.compute_done[b])   # x[b] was read by step i-2
            else:
                self.h2d.wait_stream(main)
            with torch.cuda.stream(self.h2d):
                self.x[b].copy_(h_in, non_blocking=True)
                self.in_ready[b].record(self.h2d)
            main.wait_event(self.in_ready[b])
            if i >= 2:
                main.wait_event(self.out_copied[b])          # y[b] still being downloaded
            self.layer.step(self.x[b], out=self.y[b])
            self.compute_done[b].record(main)
            self.d2h.wait_event(self.compute_done[b])
            with torch.cuda.stream(self.d2h):
                h_out.copy_(self.y[b], non_blocking=True)
                self.out_copied[b].record(self.d2h)
        main.wait_stream(self.h2d)
        main.wait_stream(self.d2h)


class SingleGpuLayer:
    """One GPU, all experts local: a single qs3_moe_layer_execute per step."""

    def __init__(self, ctx, data):
        import torch
        from qs3_b200 import ops
        self.ops, self.ctx, self.data = ops, ctx, data
        cfg = data.cfg
        self.plan = data.plan(ctx)
        dev = data.hidden.device
        self.ws = torch.empty(self.plan.layer_workspace_size(cfg.tokens, cfg.shared_inter), dtype=torch.uint8,
                              device=dev)
        self.out = torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16, device=dev)
        self.x_dev = torch.empty_like(data.hidden)
        self.ids = torch.empty((cfg.tokens, cfg.top_k), dtype=torch.int32, device=dev)
        self.graph = None
        self.launches_per_step = 0

    def step(self, hidden=None, out=None, **outputs):
        if self.graph is not None and hidden is None and out is None and not outputs:
            self.graph.replay()
            return
        d = self.data
        self.ops.moe_layer_execute(self.plan, d.hidden if hidden is None else hidden, d.router, d.gate_up,
                                   d.down, self.out if out is None else out, self.ws, router_bias=d.bias,
                                   shared=d.shared, topk_ids=self.ids, **outputs)

    def capture(self):
        """Capture one resident-input step in a CUDA graph (decode-sized steps are otherwise
        bound by the host's launch rate, not by the GPU)."""
        import torch
        for _ in range(3):
            self.step()
        torch.cuda.synchronize()
        before = self.ops.launch_count()
        self.step()
        self.launches_per_step = self.ops.launch_count() - before
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.ctx.use_current_stream()
            self.step()
        self.ctx.use_current_stream()
        self.graph = graph

    def try_capture(self):
        import torch
        try:
            self.capture()
        except Exception as exc:  # capture is an optimisation of the launch path only
            print(f"CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            self.ctx.use_current_stream()
            self.graph = None

    def profile(self, iters):
        acc = {}
        graph, self.graph = self.graph, None  # stage events are recorded by eager launches only
        try:
            for _ in range(iters):
                self.ops.profile_begin(self.ctx)
                self.step()
                for name, ms in self.ops.profile_end(self.ctx):
                    acc.setdefault(name, []).append(ms)
        finally:
            self.graph = graph
        return {k: statistics.mean(v) for k, v in acc.items()}

    def parity(self, sample=64):
        """One more eager step that also writes logits / ids / weights, compared with the CPU
        oracle: ids and permutation of all tokens, outputs of `sample` tokens."""
        import torch
        from oracle import parity
        cfg = self.data.cfg
        dev = self.out.device
        wts = torch.empty((cfg.tokens, cfg.top_k), dtype=torch.float32, device=dev)
        logits = torch.empty((cfg.tokens, cfg.experts), dtype=torch.float32, device=dev)
        graph, self.graph = self.graph, None
        try:
            self.step(topk_weights=wts, router_logits=logits)
        finally:
            self.graph = graph
        torch.cuda.synchronize()
        tables = [x.cpu().numpy() for x in self.plan.routing_tables(self.ws, cfg.tokens)]
        host = parity.host_copies(self.data)
        return parity.check_layer(host, cfg, logits=logits.cpu().numpy(), ids=self.ids.cpu().numpy(),
                                  weights=wts.cpu().numpy(),
                                  out=self.out.cpu().view(torch.uint16).numpy(), tables=tables, sample=sample)

    def _counts(self):
        import torch
        cfg = self.data.cfg
        counts = torch.bincount(self.ids.flatten().long(), minlength=cfg.experts)
        return int((counts > 0).sum().item()), int(counts.max().item())

    def roofline(self, stage_ms, hbm_gbs, peak_kind, probe=True):
        """Dominant kernel: grouped gate_up GEMM + SwiGLU. Algorithmic bytes per launch =
        gate_up weights (codes + scales) of every expert that received a row, plus the
        quantised activation rows read and the quantised SwiGLU rows written; algorithmic
        FLOPs = 2 * routes * 2I * H. The launch is bound by whichever of the two takes longer at
        its measured peak (HBM copy bandwidth / tensor-pipe ceiling of the operand format,
        measured here with an issue loop of 128 x 256 tcgen05.mma on resident tiles); `bound`,
        `achieved`, `peak`, `frac` describe that resource, the other one is reported beside it."""
        cfg = self.data.cfg
        ms = stage_ms.get("gate_up_gemm_swiglu")
        if not ms:
            return None
        hit, max_rows = self._counts()
        routes = cfg.tokens * cfg.top_k
        gu_bytes, d_bytes = self.data.weight_bytes_per_expert()
        flops = 2.0 * routes * 2 * cfg.inter * cfg.hidden
        if cfg.fp8:
            act_in = routes * (cfg.hidden + cfg.hidden // 128 * 4)
            act_out = routes * (cfg.inter + cfg.inter // 128 * 4)
            kernel, nominal, fallback_ceiling = "gemm_fp8_kernel<16, gated>", 4500.0, 3413.0
        else:
            act_in = routes * (cfg.hidden // 2 + cfg.hidden // 16)
            act_out = routes * (cfg.inter // 2 + cfg.inter // 16)
            decode = routes <= 16 * cfg.experts   # the plan's own rule for the swapped-operand kernel
            kernel = "gemm_nvfp4_swap_kernel<gated>" if decode else GATE_UP_KERNEL
            nominal, fallback_ceiling = 9000.0, 6642.0
        algo = hit * gu_bytes + act_in + act_out
        hbm_achieved = algo / (ms * 1e-3) / 1e9
        tflops = flops / (ms * 1e-3) / 1e12
        fmt = "fp8" if cfg.fp8 else "nvfp4"
        if probe:
            ceiling, ceiling_src = self.ops.tensor_peak_probe(self.ctx, fmt, 256, 20000), \
                "measured in this run: issue loop of 128 x 256 tcgen05.mma on resident tiles, every SM"
        else:
            ceiling, ceiling_src = fallback_ceiling, "issue-loop probe of an earlier run on this pool"
        t_hbm, t_tensor = algo / (hbm_gbs * 1e9), flops / (ceiling * 1e12)
        tensor_bound = t_tensor > t_hbm
        # DRAM bytes per launch: ncu's dram read + write over the algorithmic bytes, measured once per
        # kernel on a reduced case of the same layer (profiles/), scaled here by the algorithmic bytes
        traffic = TRAFFIC_RATIO[kernel] * algo
        out = {"bound": "tensor" if tensor_bound else "hbm",
               "achieved": tflops if tensor_bound else hbm_achieved,
               "peak": ceiling if tensor_bound else hbm_gbs,
               "unit": "TFLOP/s" if tensor_bound else "GB/s",
               "frac": (tflops / ceiling) if tensor_bound else (hbm_achieved / hbm_gbs),
               "peak_source": ceiling_src if tensor_bound else f"{peak_kind} copy bandwidth",
               "traffic": traffic,
               "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, ratio to algorithmic bytes "
                                 "measured once per kernel on a reduced case and scaled to this launch",
               "kernel": kernel, "kernel_ms": ms, "algorithmic_bytes": algo, "algorithmic_flops": flops,
               "experts_hit": hit, "max_rows_per_expert": max_rows,
               "time_at_hbm_peak_ms": t_hbm * 1e3, "time_at_tensor_ceiling_ms": t_tensor * 1e3,
               "hbm_gbs": hbm_achieved, "hbm_frac": hbm_achieved / hbm_gbs,
               "tensor_tflops": tflops, "tensor_ceiling_tflops": ceiling,
               "tensor_frac_of_measured_ceiling": tflops / ceiling,
               "tensor_frac_of_nominal": tflops / nominal}
        ms2 = stage_ms.get("down_gemm")
        if ms2:
            algo2 = hit * d_bytes + act_out + routes * cfg.hidden * 2
            flops2 = 2.0 * routes * cfg.inter * cfg.hidden
            out["down_gemm"] = {"kernel_ms": ms2, "algorithmic_bytes": algo2,
                                "achieved": algo2 / (ms2 * 1e-3) / 1e9,
                                "frac": algo2 / (ms2 * 1e-3) / 1e9 / hbm_gbs,
                                "tensor_tflops": flops2 / (ms2 * 1e-3) / 1e12,
                                "tensor_frac_of_measured_ceiling": flops2 / (ms2 * 1e-3) / 1e12 / ceiling}
        return out

    def stage_rooflines(self, stage_ms, hbm_gbs):
        """HBM fractions of the routing, permute and combine kernels (algorithmic bytes per stage /
        the stage's CUDA-event time / the measured copy bandwidth)."""
        cfg = self.data.cfg
        t, h, e, k = cfg.tokens, cfg.hidden, cfg.experts, cfg.top_k
        r = t * k
        row = (h // 2 + h // 16) if cfg.nvfp4 else (h + h // 32) if cfg.fp8 else 2 * h
        algo = {
            "router_logits_gemm": t * h * 2 + e * h * 2 + t * e * 4,
            "router_topk": t * e * 4 + r * 8,
            "route_sort": r * 4 + r * 16,
            # tokens read once as bf16 and written once quantised (side stream), then R rows gathered
            "gather_quantize": (t * h * 2 + t * row if cfg.nvfp4 else 0) + 2 * r * row,
            "combine": r * h * 2 + t * h * 2 + (2 * t * h * 2 if cfg.shared_inter else 0),
        }
        out = []
        for name, nbytes in algo.items():
            ms = stage_ms.get(name)
            if ms:
                gbs = nbytes / (ms * 1e-3) / 1e9
                out.append({"name": name, "ms": ms, "bytes": nbytes, "gbs": gbs, "frac_hbm": gbs / hbm_gbs})
        return out


# the library's own dispatch rule for the NVFP4 prefill gate_up GEMM (QS3_NVFP4_PAIR=0 selects the
# single-CTA resident-A kernel); the bench workloads satisfy the pair kernel's shape rules
GATE_UP_KERNEL = ("gemm_tc_astat_kernel<gated, swiglu_nvfp4>" if os.environ.get("QS3_NVFP4_PAIR") == "0"
                  else "gemm_nvfp4_pair_kernel<gated, swiglu_nvfp4>")
TRAFFIC_RATIO = {"gemm_nvfp4_pair_kernel<gated, swiglu_nvfp4>": 1.07,
                 "gemm_tc_astat_kernel<gated, swiglu_nvfp4>": 1.02,
                 "gemm_nvfp4_swap_kernel<gated>": 1.00,
                 "gemm_fp8_kernel<16, gated>": 1.02}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill_nvfp4", choices=["prefill_nvfp4", "decode_fp8", "decode_nvfp4"],
                    help="N = 1 only: the FP8 decode batch (64 tokens, 128 experts, top-8) or a 128-token decode "
                         "batch of the NVFP4 layer instead of the headline layer")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="N > 1: how the experts are assigned to ranks")
    ap.add_argument("--hot-experts", type=int, default=32,
                    help="N > 1, balanced placement: replicate this many of the hottest experts on every rank")
    ap.add_argument("--no-graph", action="store_true",
                    help="N = 1: launch the resident-input steps eagerly instead of replaying one CUDA graph "
                         "(the e2e leg is always eager)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled check against the CPU oracle")
    ap.add_argument("--no-secondary", action="store_true", help="N = 1: skip the decode workloads after the headline")
    ap.add_argument("--no-hybrid", action="store_true",
                    help="N = 1: skip the 48-layer hybrid decode loop among the secondary workloads (it holds "
                         "about 50 GB of random weights and takes the longest to set up)")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="GPU time the back-to-back blocks of `--steps` steps must cover at least")
    ap.add_argument("--kernels-only", action="store_true",
                    help="only the device-timed loop (for profiler captures; prints no valid bench line)")
    ap.add_argument("--tokens", type=int, default=0, help="reduced token count, profiler captures only")
    ap.add_argument("--experts", type=int, default=0, help="reduced expert count, profiler captures only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    elif args.gpus != 1:
        raise SystemExit("launch N > 1 with torch.distributed.run (one process per GPU)")
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
