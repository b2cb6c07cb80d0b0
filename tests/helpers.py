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


# ------------------------------------------------------- synthetic checkpoints ---

_ST_ITEMSIZE = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1,
                "U16": 2, "U32": 4, "U64": 8, "BOOL": 1, "F8_E4M3": 1, "F8_E5M2": 1}


def write_safetensors(path, tensors, metadata=None):
    """Minimal safetensors writer for test fixtures: ``tensors`` maps a name to
    (dtype spelling, shape, numpy array or bytes); data is laid out in the given order."""
    import json
    import struct
    header, blobs, at = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, shape, data) in tensors.items():
        raw = data if isinstance(data, (bytes, bytearray)) else np.ascontiguousarray(data).tobytes()
        assert len(raw) == int(np.prod(shape, dtype=np.int64)) * _ST_ITEMSIZE[dtype], name
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def write_raw_safetensors(path, header_text, data=b""):
    """A shard with an arbitrary (possibly malformed) header, for the rejection tests."""
    import struct
    raw = header_text if isinstance(header_text, bytes) else header_text.encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)) + raw + data)


def moe_checkpoint_tensors(prefix, d, *, nvfp4, shared_nvfp4=True, transposed=False, seed=0):
    """Tensors of one MoE layer in the two checkpoint conventions, from the bf16 arrays of
    `make_moe_inputs`. Returns (tensors for `write_safetensors`, reference dict). For NVFP4
    every projection is quantised on its own (own global scale), as split checkpoints have it;
    the reference dict holds the fused arrays a loader must produce."""
    rng = np.random.default_rng(seed)
    e, two_i, h = d["gate_up"].shape
    i = two_i // 2
    t = {prefix + "gate.weight": ("BF16", (e, h), d["router"])}
    ref = {}
    shared = "sh_gate_up" in d

    def nvfp4_proj(stem, w, input_scale):
        packed, lin, _tiled, g = orc.nvfp4_quantize_weight(w[None], False)
        t[stem + ".weight"] = ("U8", packed.shape[1:], packed[0])
        t[stem + ".weight_scale"] = ("F8_E4M3", lin.shape[1:], lin[0])
        t[stem + ".weight_scale_2"] = ("F32", (), np.float32(g[0]))
        t[stem + ".input_scale"] = ("F32", (1,), np.array([input_scale], np.float32))
        return packed[0], lin[0], float(g[0])

    if nvfp4:
        gu_p = np.empty((e, 2 * i, h // 2), np.uint8)
        gu_s = np.empty((e, 2 * i, h // 16), np.uint8)
        gu_g = np.empty((2, e), np.float32)
        d_p = np.empty((e, h, i // 2), np.uint8)
        d_s = np.empty((e, h, i // 16), np.uint8)
        d_g = np.empty(e, np.float32)
        in1 = (0.5 + rng.random(e) * 0.5).astype(np.float32) * 2.0 ** -6   # per-expert activation scales
        in2 = (0.5 + rng.random(e) * 0.5).astype(np.float32) * 2.0 ** -10
        for x in range(e):
            stem = f"{prefix}experts.{x}."
            gu_p[x, :i], gu_s[x, :i], gu_g[0, x] = nvfp4_proj(stem + "gate_proj", d["gate_up"][x, :i], in1[x])
            gu_p[x, i:], gu_s[x, i:], gu_g[1, x] = nvfp4_proj(stem + "up_proj", d["gate_up"][x, i:], in1[x] * 0.9)
            d_p[x], d_s[x], d_g[x] = nvfp4_proj(stem + "down_proj", d["down"][x], in2[x])
        ref.update(gu=(gu_p, gu_s, gu_g), d=(d_p, d_s, d_g), act=float(in1.max()), act2=float(in2.max()))
    else:
        gu, dn = d["gate_up"], d["down"]
        if transposed:
            gu, dn = np.ascontiguousarray(gu.transpose(0, 2, 1)), np.ascontiguousarray(dn.transpose(0, 2, 1))
        t[prefix + "experts.gate_up_proj"] = ("BF16", gu.shape, gu)
        t[prefix + "experts.down_proj"] = ("BF16", dn.shape, dn)
    if shared:
        s = d["sh_gate_up"].shape[1] // 2
        stem = prefix + "shared_expert."
        if nvfp4 and shared_nvfp4:
            sp = np.empty((1, 2 * s, h // 2), np.uint8)
            ss = np.empty((1, 2 * s, h // 16), np.uint8)
            sg = np.empty(2, np.float32)
            sp[0, :s], ss[0, :s], sg[0] = nvfp4_proj(stem + "gate_proj", d["sh_gate_up"][0, :s], ref["act"] * 0.7)
            sp[0, s:], ss[0, s:], sg[1] = nvfp4_proj(stem + "up_proj", d["sh_gate_up"][0, s:], ref["act"] * 0.7)
            ref["act2"] = float(np.float32(ref["act2"] * 1.25))   # the shared expert's input scale is the largest
            dp, ds, dg = nvfp4_proj(stem + "down_proj", d["sh_down"][0], ref["act2"])
            ref.update(sh_gu=(sp, ss, sg), sh_d=(dp[None], ds[None], np.array([dg], np.float32)))
        else:
            t[stem + "gate_proj.weight"] = ("BF16", (s, h), d["sh_gate_up"][0, :s])
            t[stem + "up_proj.weight"] = ("BF16", (s, h), d["sh_gate_up"][0, s:])
            t[stem + "down_proj.weight"] = ("BF16", (h, s), d["sh_down"][0])
        t[prefix + "shared_expert_gate.weight"] = ("BF16", (1, h), d["sh_gate"])
    return t, ref
