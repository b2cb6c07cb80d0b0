"""Shared helpers of the test-suite: seeded synthetic inputs with the shapes and
value distributions of the benchmark configurations, known-answer case builders,
and error metrics. numpy only; bf16 tensors are uint16 bit patterns."""
from __future__ import annotations

import math

import numpy as np

from oracle import binding as orc


def bf16(x):
    return orc.f32_to_bf16(np.asarray(x, dtype=np.float32))


def f32(b):
    return orc.bf16_to_f32(b)


def silu(x):
    return x / (1.0 + math.exp(-x))


def eval_expected(expr):
    return float(eval(expr, {"silu": silu})) if isinstance(expr, str) else float(expr)


def parse_floats(values):
    return np.array([float(v) for v in values], dtype=np.float32)


def rel_l2(got_bf16, want_bf16):
    g = f32(got_bf16).astype(np.float64)
    w = f32(want_bf16).astype(np.float64)
    return float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30))


def max_abs(got_bf16, want_bf16):
    return float(np.max(np.abs(f32(got_bf16).astype(np.float64) - f32(want_bf16).astype(np.float64))))


def moe_case_arrays(case):
    """Dense arrays of one hand-written MoE case of tests/golden/reference_cases.json."""
    t, h, i, e, k = case["tokens"], case["hidden"], case["intermediate"], case["experts"], case["top_k"]
    hidden = np.zeros((t, h), np.float32)
    for r, c, v in case["hidden_nonzero"]:
        hidden[r, c] = v
    gate_up = np.zeros((e, 2 * i, h), np.float32)
    for ex, r, c, v in case["gate_up_nonzero"]:
        gate_up[ex, r, c] = v
    down = np.zeros((e, h, i), np.float32)
    for ex, r, c, v in case["down_nonzero"]:
        down[ex, r, c] = v
    expected = np.zeros((t, h), np.float32)
    for r, c, expr in case["expected_nonzero"]:
        expected[r, c] = eval_expected(expr)
    ids = np.array(case["topk_ids"], np.int32).reshape(t, k)
    w = np.array(case["topk_weights"], np.float32).reshape(t, k)
    return bf16(hidden), ids, w, bf16(gate_up), bf16(down), expected


def zipf_bias(num_experts, rng, s=1.1):
    """Per-expert additive logit bias -s * ln(1 + rank), ranks assigned by a seeded
    permutation, so that expert load follows a Zipf-like law."""
    perm = rng.permutation(num_experts)
    return (-s * np.log1p(perm.astype(np.float64))).astype(np.float32)


def make_moe_inputs(seed, tokens, hidden, experts, inter, shared_inter=0, weight_std=0.02):
    """Activations ~ N(0,1), all weights ~ N(0, 0.02), rounded to bf16."""
    rng = np.random.default_rng(seed)
    out = {
        "hidden": bf16(rng.standard_normal((tokens, hidden), dtype=np.float32)),
        "router": bf16(rng.standard_normal((experts, hidden), dtype=np.float32) * weight_std),
        "gate_up": bf16(rng.standard_normal((experts, 2 * inter, hidden), dtype=np.float32) * weight_std),
        "down": bf16(rng.standard_normal((experts, hidden, inter), dtype=np.float32) * weight_std),
        "rng": rng,
    }
    if shared_inter:
        out["sh_gate_up"] = bf16(rng.standard_normal((1, 2 * shared_inter, hidden), dtype=np.float32) * weight_std)
        out["sh_down"] = bf16(rng.standard_normal((1, hidden, shared_inter), dtype=np.float32) * weight_std)
        out["sh_gate"] = bf16(rng.standard_normal((1, hidden), dtype=np.float32) * weight_std)
    return out


# ------------------------------------------------------------ device helpers ---

def to_dev(a, kind=None):
    """numpy -> torch device tensor; uint16 arrays become bf16 unless kind == 'raw'."""
    import torch
    a = np.ascontiguousarray(a)
    t = torch.from_numpy(a)
    if a.dtype == np.uint16 and kind != "raw":
        t = t.view(torch.bfloat16)
    return t.cuda()


def to_np(t):
    """torch device tensor -> numpy; bf16 tensors come back as uint16 bit patterns."""
    import torch
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().copy()
    return t.numpy().copy()
