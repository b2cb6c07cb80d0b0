"""Sampled parity check of one whole MoE layer against the CPU oracle.

Test infrastructure, like everything under ``oracle/``: the GPU tests and the check
that ``bench.py`` runs once after its timed loops call this; the library never does.
Everything here is numpy; callers hand over host copies of what the device produced.

What is compared, for a layer of T tokens:

* expert ids of ALL tokens, bit for bit, against ``router_topk`` run on the logits the
  device wrote (routing is exact on identical logits; the logits themselves are
  compared with the oracle's GEMM on the sampled tokens, f32 summation order differs);
* router weights of all tokens, absolute tolerance 1e-5 (upstream's own bound,
  tests_cuda_qscu_gdn_router.inc:1031-1036);
* ``counts``, ``indptr``, ``route_rows``, ``row_tokens`` of all routes, bit for bit,
  against ``route_sort`` (stable in route index) when the caller passes the tables;
* the layer output of a SAMPLE of tokens against the oracle's layer restricted to
  those tokens (its ``token_list`` argument): rel-L2 <= 1e-2 and
  max-abs <= 2^-5 * max|ref| (2^-6 for bf16 plans). The sample always holds tokens
  routed to the largest expert (first and last rows, i.e. first and last row tile),
  to experts that received a single row, to small experts, and random others.
"""
from __future__ import annotations

import numpy as np

from . import binding as orc


def host_copies(data):
    """numpy copies of a ``qs3_b200.workload.LayerData`` (weights in the declared linear layout)."""
    import torch

    def triple(q):
        if hasattr(q, "codes"):
            return (q.codes.cpu().numpy(), q.scale.cpu().numpy())
        if hasattr(q, "packed"):
            return (q.packed.cpu().numpy(), q.scale_linear.cpu().numpy(), q.global_scale.cpu().numpy())
        return q.cpu().view(torch.uint16).numpy()

    host = {
        "hidden": data.hidden.cpu().view(torch.uint16).numpy(),
        "router": data.router.cpu().view(torch.uint16).numpy(),
        "bias": None if data.bias is None else data.bias.cpu().numpy(),
        "gu": triple(data.gate_up), "d": triple(data.down), "shared": None,
    }
    if data.shared is not None:
        host["shared"] = dict(gu=triple(data.shared.gate_up), d=triple(data.shared.down),
                              gate_w=data.shared.gate_weight.cpu().view(torch.uint16).numpy())
    return host


def oracle_layer(host, cfg, tokens, ids=None, weights=None):
    """Whole layer on the host cores for the listed tokens; returns (bf16 bit patterns, ids).
    With ``ids`` / ``weights`` (arrays over ALL tokens) the routing is taken from them."""
    tokens = np.asarray(tokens, dtype=np.int64)
    hid = host["hidden"][tokens]
    if ids is None:
        logits = orc.gemm_bf16(hid, host["router"], "f32")
        sel_ids, sel_w = orc.router_topk(logits, cfg.top_k, 0, True, 1.0, host["bias"])
    else:
        sel_ids, sel_w = ids[tokens], weights[tokens]
    if getattr(cfg, "fp8", False):
        hc, hs = orc.fp8_quantize_act(hid)
        return orc.moe_fp8(hc, hs, sel_ids, sel_w, host["gu"], host["d"]), sel_ids
    if cfg.nvfp4:
        hp, hs = orc.nvfp4_quantize_act(hid, 1.0)
        return orc.moe_nvfp4(hp, hs, sel_ids, sel_w, host["gu"], host["d"], shared=host["shared"],
                             hidden_bf16=hid), sel_ids
    out = orc.moe_bf16(hid, sel_ids, sel_w, host["gu"], host["d"])
    if host["shared"] is not None:
        sh = host["shared"]
        out = orc.shared_expert_bf16(hid, sh["gu"], sh["d"], sh["gate_w"], out)
    return out, sel_ids


def pick_tokens(ids, num_experts, n, seed=0):
    """``n`` distinct token indices covering the regimes a ragged grouped GEMM has: the largest
    experts' first and last rows, single-row experts, small experts, random tokens."""
    t, k = ids.shape
    rng = np.random.default_rng(seed)
    flat = ids.reshape(-1)
    counts = np.bincount(flat[(flat >= 0) & (flat < num_experts)], minlength=num_experts)
    chosen: list[int] = []

    def add(tok):
        tok = int(tok)
        if tok not in chosen and len(chosen) < n:
            chosen.append(tok)

    def tokens_of(e):
        return np.nonzero((ids == e).any(axis=1))[0]

    order = np.argsort(-counts, kind="stable")
    for e in order[:4]:                      # largest experts: first / last row tile, and the middle
        if counts[e] == 0:
            break
        toks = tokens_of(e)
        for tok in (toks[0], toks[-1], toks[len(toks) // 2], toks[-min(2, len(toks))]):
            add(tok)
    singles = np.nonzero(counts == 1)[0]
    for e in singles[:8]:
        add(tokens_of(e)[0])
    small = np.nonzero((counts >= 2) & (counts <= 16))[0]
    for e in small[:8]:
        add(tokens_of(e)[-1])
    ragged = np.nonzero((counts > 128) & (counts % 128 != 0))[0]
    for e in ragged[:6]:                     # last (partial) tile of multi-tile experts
        add(tokens_of(e)[-1])
    while len(chosen) < min(n, t):
        add(rng.integers(0, t))
    return np.array(sorted(chosen), dtype=np.int64)


def check_layer(host, cfg, *, logits, ids, weights, out, tables=None, table_range=None, sample=64, seed=0,
                out_rows=None):
    """Compare one executed layer with the oracle. ``logits`` f32 [T, E], ``ids`` i32 [T, K],
    ``weights`` f32 [T, K], ``out`` bf16 bit patterns [T, H] as the device wrote them;
    ``tables`` = (counts, indptr, route_rows, row_tokens) of the plan that owns experts
    ``table_range`` = (first, count) (default: all). Returns a dict of findings; ``ok`` is the
    conjunction of every bound stated in the module docstring."""
    t, k = ids.shape
    res = {"tokens": int(t), "tokens_checked": 0}
    ids_ref, w_ref = orc.router_topk(logits, k, 0, True, 1.0, host["bias"])
    res["ids_exact"] = bool(np.array_equal(ids, ids_ref))
    res["ids_mismatches"] = int((ids != ids_ref).sum())
    res["weights_max_abs"] = float(np.max(np.abs(weights - w_ref))) if t else 0.0
    ok = res["ids_exact"] and res["weights_max_abs"] <= 1e-5
    if tables is not None:
        first, count = table_range if table_range is not None else (0, cfg.experts)
        counts, indptr, route_rows, row_tokens = (np.asarray(x) for x in tables[:4])
        c_ref, p_ref, rr_ref, rt_ref, _ = orc.route_sort(ids, weights, first, count)
        n_rows = int(p_ref[-1])
        res["tables_exact"] = bool(np.array_equal(counts, c_ref) and np.array_equal(indptr, p_ref)
                                   and np.array_equal(route_rows, rr_ref)
                                   and np.array_equal(row_tokens[:n_rows], rt_ref))
        res["experts_hit"] = int((c_ref > 0).sum())
        res["max_rows_per_expert"] = int(c_ref.max()) if count else 0
        ok = ok and res["tables_exact"]
    tokens = pick_tokens(ids, cfg.experts, sample, seed)
    ref_logits = orc.gemm_bf16(host["hidden"][tokens], host["router"], "f32")
    res["logits_max_abs"] = float(np.max(np.abs(ref_logits - logits[tokens])))
    ok = ok and res["logits_max_abs"] <= 1e-4
    ref, _ = oracle_layer(host, cfg, tokens, ids=ids, weights=weights)
    got = out[tokens] if out_rows is None else out[out_rows[tokens]]
    g = orc.bf16_to_f32(got).astype(np.float64)
    w = orc.bf16_to_f32(ref).astype(np.float64)
    res["rel_l2"] = float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30))
    res["max_abs"] = float(np.max(np.abs(g - w)))
    res["max_abs_bound"] = float(2.0 ** (-5 if (cfg.nvfp4 or getattr(cfg, "fp8", False)) else -6)
                                 * np.max(np.abs(w)))
    # per-token rel-L2: a single bad row must not hide in the average
    per_tok = np.linalg.norm(g - w, axis=1) / np.maximum(np.linalg.norm(w, axis=1), 1e-30)
    res["rel_l2_worst_token"] = float(per_tok.max())
    res["tokens_checked"] = int(tokens.size)
    ok = ok and res["rel_l2"] <= 1e-2 and res["max_abs"] <= res["max_abs_bound"] and res["rel_l2_worst_token"] <= 3e-2
    res["ok"] = bool(ok)
    return res
