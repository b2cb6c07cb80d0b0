"""Pins the CPU oracle against the known-answer cases of the upstream CUDA tests
(tests/golden/reference_cases.json) before anything else trusts it."""
import math

import numpy as np

from helpers import bf16, f32, moe_case_arrays, parse_floats


def _router_case(oracle, case, logits_bf16=False):
    logits = parse_floats(case["logits"]).reshape(case["num_tokens"], case["num_experts"])
    if logits_bf16:
        logits = f32(bf16(logits))
    return logits, oracle.router_topk(logits, case["top_k"], case["score"], bool(case["renormalize"]),
                                      case["scale"])


def test_router_softmax_ties(oracle, golden):
    case = golden["router_softmax_ties"]
    logits, (ids, w) = _router_case(oracle, case)
    assert ids.tolist() == case["expected_ids"]
    # closed form: softmax over the row, renormalised over the selected three, times scale
    for t in range(2):
        p = np.exp(logits[t].astype(np.float64) - logits[t].max())
        p /= p.sum()
        sel = p[ids[t]]
        want = sel / sel.sum() * case["scale"]
        assert np.allclose(w[t], want, atol=case["weight_tolerance"])


def test_router_sigmoid_bf16(oracle, golden):
    case = golden["router_sigmoid_bf16"]
    logits, (ids, w) = _router_case(oracle, case, logits_bf16=True)
    assert ids.tolist() == case["expected_ids"]
    want = case["scale"] / (1.0 + math.exp(-1.0))
    assert np.allclose(w[0], [want, want], atol=case["weight_tolerance"])


def test_router_nonfinite(oracle, golden):
    case = golden["router_nonfinite"]
    _, (ids, w) = _router_case(oracle, case)
    assert ids.tolist() == case["expected_ids"]
    assert np.all(np.isfinite(w))
    assert np.allclose(w, case["expected_weights"], atol=case["weight_tolerance"])


def test_router_unfilled_slots(oracle):
    # only NaN / -inf logits: nothing qualifies, slots keep id = slot index and weight 0
    # (upstream qscu.cu:945-949)
    logits = np.array([[np.nan, -np.inf, np.nan, 1.0]], np.float32)
    ids, w = oracle.router_topk(logits, 3, 0, True, 1.0)
    assert ids.tolist() == [[3, 1, 2]]
    assert w[0, 1] == 0.0 and w[0, 2] == 0.0


def test_moe_known_answers(oracle, golden):
    for name in ("moe_staged_grouped_gemm", "moe_top2_weighted_accumulation"):
        case = golden[name]
        hidden, ids, w, gate_up, down, expected = moe_case_arrays(case)
        out = f32(oracle.moe_bf16(hidden, ids, w, gate_up, down))
        assert np.max(np.abs(out - expected)) <= case["tolerance"], name
        # everything the case does not name stays exactly zero
        assert np.all(out[expected == 0.0] == 0.0), name


def test_silu_and_mul(oracle, golden):
    case = golden["silu_and_mul"]
    gate, up = bf16(case["gate"]), bf16(case["up"])
    out = f32(oracle.silu_and_mul_bf16(gate, up))
    g, u = f32(gate).astype(np.float64), f32(up).astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    assert np.max(np.abs(out - want)) <= case["tolerance"]


def test_shared_expert_gate_add(oracle, golden):
    case = golden["shared_expert_gate_add"]
    rows, hidden = case["rows"], case["hidden"]
    shared = bf16(case["shared"]).reshape(rows, hidden)
    out0 = bf16(case["out"]).reshape(rows, hidden)
    for gate in (np.array(case["gate"], np.float32), f32(bf16(case["gate"]))):
        out = f32(oracle.shared_gate_add_bf16(gate, shared, out0))
        sig = 1.0 / (1.0 + np.exp(-gate.astype(np.float64)))
        want = f32(out0) + sig[:, None] * f32(shared)
        assert np.max(np.abs(out - want)) <= case["tolerance"]


def test_route_sort_is_stable_and_consistent(oracle):
    rng = np.random.default_rng(3)
    t, k, e = 37, 4, 11
    ids = rng.integers(0, e, size=(t, k), dtype=np.int32)
    ids[0] = [2, 2, 2, 5]  # duplicate routes of one token accumulate (test.cu:1586)
    w = rng.random((t, k), dtype=np.float32)
    counts, indptr, route_rows, row_tokens, row_scales = oracle.route_sort(ids, w, 0, e)
    assert counts.sum() == t * k and indptr[-1] == t * k
    assert np.array_equal(counts, np.bincount(ids.ravel(), minlength=e))
    order = np.argsort(ids.ravel(), kind="stable")
    assert np.array_equal(route_rows[order], np.arange(t * k))
    assert np.array_equal(row_tokens, order // k)
    assert np.array_equal(row_scales, w.ravel()[order])
    # expert-parallel view: only experts [4, 8) are local
    counts2, indptr2, rows2, tok2, _ = oracle.route_sort(ids, w, 4, 4)
    local = (ids.ravel() >= 4) & (ids.ravel() < 8)
    assert counts2.sum() == local.sum() and np.all(rows2[~local] == -1)
    assert np.array_equal(np.sort(rows2[local]), np.arange(local.sum()))


def test_bf16_round_to_nearest_even(oracle):
    # upstream src/model.rs:3000-3004: bits + 0x7FFF + lsb
    cases = {1.0: 0x3F80, 1.00390625: 0x3F80, 1.01171875: 0x3F82, -2.5: 0xC020, 0.0: 0x0000}
    for v, want in cases.items():
        assert int(bf16([v])[0]) == want
        assert oracle.lib().qs3o_f32_to_bf16(v) == want


def test_fp4_fp8_codecs(oracle):
    lib = oracle.lib()
    # e2m1 grid and tie-to-even midpoints
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c, v in enumerate(grid):
        assert lib.qs3o_e2m1_to_f32(c) == v and lib.qs3o_f32_to_e2m1(v) == c
        assert lib.qs3o_f32_to_e2m1(-v) == (c | 8 if v != 0.0 else 8)
    for mid, code in ((0.25, 0), (0.75, 2), (1.25, 2), (1.75, 4), (2.5, 4), (3.5, 6), (5.0, 6), (100.0, 7)):
        assert lib.qs3o_f32_to_e2m1(mid) == code
    # e4m3: exact round trip of every finite non-negative code, saturation, subnormals
    for c in range(0x7F):
        v = lib.qs3o_e4m3_to_f32(c)
        assert lib.qs3o_f32_to_e4m3(v) == c
    assert lib.qs3o_e4m3_to_f32(0x7E) == 448.0 and lib.qs3o_f32_to_e4m3(1e9) == 0x7E
    assert lib.qs3o_e4m3_to_f32(0x01) == 2.0 ** -9 and lib.qs3o_f32_to_e4m3(2.0 ** -10) == 0
    assert lib.qs3o_f32_to_e4m3(1.5 * 2.0 ** -9) == 2  # tie -> even


def test_e4m3_codec_against_torch_float8(oracle):
    """The oracle's e4m3 codec pinned to an implementation outside this repository:
    torch.float8_e4m3fn decodes all 256 codes to the same values (the two NaN codes aside) and
    rounds a dense sweep of floats, every midpoint between neighbouring e4m3 values included
    (ties to even), to the same codes. Above 448 the oracle saturates (its quantisers never
    produce NaN) where torch's cast does not, so the sweep stops at 448."""
    import torch
    lib = oracle.lib()
    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    got = oracle.e4m3_to_f32(codes)
    finite = ~np.isnan(want)
    assert finite.sum() == 254 and np.array_equal(got[finite], want[finite])
    pos = np.sort(want[finite & (want >= 0)])
    mids = (pos[:-1] + pos[1:]) / 2.0
    rng = np.random.default_rng(11)
    sweep = np.concatenate([pos, mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)),
                            np.exp(rng.uniform(np.log(2.0 ** -11), np.log(448.0), 20000)),
                            rng.uniform(0.0, 448.0, 5000)]).astype(np.float32)
    sweep = np.concatenate([sweep, -sweep])
    t_codes = torch.from_numpy(sweep).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    o_codes = np.array([lib.qs3o_f32_to_e4m3(float(v)) for v in sweep], dtype=np.uint8)
    # -0.0 and +0.0 encode alike up to the sign bit in both
    assert np.array_equal(o_codes & 0x7F, t_codes & 0x7F)
    nz = (o_codes & 0x7F) != 0
    assert np.array_equal(o_codes[nz], t_codes[nz])


def test_e2m1_codec_against_the_published_value_set(oracle):
    """e2m1 (OCP microscaling FP4: 1 sign, 2 exponent, 1 mantissa bit, bias 1, no inf / NaN):
    the sixteen values are +-{0, 0.5, 1, 1.5, 2, 3, 4, 6}, computed here from the bit fields of
    the format definition rather than from the oracle's table; encoding rounds to nearest with
    ties to the even mantissa and saturates at 6."""
    lib = oracle.lib()

    def decode(c):
        sign = -1.0 if c & 8 else 1.0
        exp, man = (c >> 1) & 3, c & 1
        return sign * (man * 0.5 if exp == 0 else (1.0 + 0.5 * man) * 2.0 ** (exp - 1))

    values = [decode(c) for c in range(16)]
    assert sorted(set(abs(v) for v in values)) == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c in range(16):
        assert lib.qs3o_e2m1_to_f32(c) == values[c]
    pos = values[:8]
    rng = np.random.default_rng(12)
    sweep = np.concatenate([rng.uniform(0, 8, 4000), [(a + b) / 2 for a, b in zip(pos[:-1], pos[1:])]])
    for v in sweep:
        d = [abs(v - p) for p in pos]
        best = min(d)
        ties = [i for i, x in enumerate(d) if x == best]
        want = ties[0] if len(ties) == 1 else [i for i in ties if i % 2 == 0][0]   # even mantissa bit
        assert lib.qs3o_f32_to_e2m1(float(np.float32(v))) == want
        assert lib.qs3o_f32_to_e2m1(-float(np.float32(v))) == want | 8


def test_nvfp4_quantise_round_trip(oracle):
    rng = np.random.default_rng(5)
    x = bf16(rng.standard_normal((8, 64), dtype=np.float32))
    packed, scale = oracle.nvfp4_quantize_act(x, 1.0)
    deq = oracle.nvfp4_dequantize(packed, scale)
    # block-wise error bound: half an e2m1 step (<= 1 at the top of the grid) times the scale
    s = np.repeat(oracle.e4m3_to_f32(scale), 16, axis=-1)
    assert np.all(np.abs(deq - f32(x)) <= s * 1.0 + 1e-6)
    # exactly representable data survives: codes * power-of-two scale
    y = np.tile(np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -6, -4, -3, -2, -1.5, -1, -.5, 0], np.float32), (1, 4))
    p2, s2 = oracle.nvfp4_quantize_act(bf16(y), 1.0)
    assert np.array_equal(oracle.nvfp4_dequantize(p2, s2), y)


def test_tiled_scale_layout_is_a_bijection(oracle):
    for rows, k, gated in ((256, 256, 0), (128, 512, 0), (1024, 2048, 512)):
        idx = oracle.tiled_scale_index(rows, k, gated)
        assert idx.min() == 0 and idx.max() == oracle.tiled_scale_bytes(rows, k) - 1
        assert np.unique(idx).size == idx.size
        for r, kb in ((0, 0), (33, 5), (rows - 1, k // 16 - 1)):
            tr = oracle.lib().qs3o_gated_tiled_row(r, gated) if gated else r
            assert idx[r, kb] == oracle.lib().qs3o_tiled_scale_offset(tr, kb, k)


def test_fp8_quantise_round_trip(oracle):
    rng = np.random.default_rng(6)
    x = bf16(rng.standard_normal((5, 256), dtype=np.float32))
    codes, scale = oracle.fp8_quantize_act(x)
    # the group maximum maps onto the top of the e4m3 grid and the relative error of a
    # normal e4m3 value is at most 2^-4
    deq = oracle.fp8_dequantize(codes, scale)
    amax = np.abs(f32(x)).reshape(5, 2, 128).max(axis=-1)
    assert np.allclose(scale, amax / 448.0, rtol=1e-6)
    assert np.all(np.abs(deq - f32(x)) <= np.abs(f32(x)) * 2.0 ** -4 + np.repeat(scale, 128, axis=-1) * 2.0 ** -9)
    # all-zero group: floor scale, zero codes
    z = np.zeros((1, 128), np.uint16)
    cz, sz = oracle.fp8_quantize_act(z)
    assert not cz.any() and sz[0, 0] == np.float32(1e-30)
    # weights: one scale per 128 x 128 block, a partial last row block included
    w = bf16(rng.standard_normal((2, 192, 256), dtype=np.float32) * 0.02)
    cw, sw = oracle.fp8_quantize_weight(w)
    assert sw.shape == (2, 2, 2)
    assert np.isclose(sw[1, 1, 0], np.abs(f32(w[1, 128:, :128])).max() / 448.0, rtol=1e-6)
    dq = oracle.fp8_dequantize(cw, sw)
    assert np.linalg.norm(dq - f32(w)) / np.linalg.norm(f32(w)) < 0.04


def test_fp8_moe_matches_dequantised_float64(oracle):
    """The FP8 chain against plain float64 algebra on the dequantised operands, with the
    oracle's own intermediate quantisation applied through its quantiser."""
    rng = np.random.default_rng(7)
    t, h, i, e, k = 6, 256, 128, 4, 2
    hidden = bf16(rng.standard_normal((t, h), dtype=np.float32))
    gu = bf16(rng.standard_normal((e, 2 * i, h), dtype=np.float32) * 0.05)
    dn = bf16(rng.standard_normal((e, h, i), dtype=np.float32) * 0.05)
    ids = np.stack([rng.permutation(e)[:k] for _ in range(t)]).astype(np.int32)
    ids[0, 1] = -1  # an unfilled slot is skipped
    w = rng.random((t, k)).astype(np.float32)
    hc, hs = oracle.fp8_quantize_act(hidden)
    guq, dnq = oracle.fp8_quantize_weight(gu), oracle.fp8_quantize_weight(dn)
    out = f32(oracle.moe_fp8(hc, hs, ids, w, guq, dnq))
    x = oracle.fp8_dequantize(hc, hs).astype(np.float64)
    gu_d = oracle.fp8_dequantize(*guq).astype(np.float64)
    dn_d = oracle.fp8_dequantize(*dnq).astype(np.float64)
    want = np.zeros((t, h))
    for tok in range(t):
        for j in range(k):
            ex = ids[tok, j]
            if ex < 0:
                continue
            y1 = gu_d[ex] @ x[tok]
            act = (y1[:i] / (1.0 + np.exp(-y1[:i])) * y1[i:]).astype(np.float32)
            # quantise the f32 activation with the same rule (group of 128 == whole row here)
            s = max(np.abs(act).max() / np.float32(448.0), np.float32(1e-30))
            q = np.array([oracle.lib().qs3o_e4m3_to_f32(oracle.lib().qs3o_f32_to_e4m3(float(np.float32(v) * (np.float32(1.0) / s))))
                          for v in act], np.float64) * float(s)
            want[tok] += float(w[tok, j]) * (dn_d[ex] @ q)
    assert np.linalg.norm(out - want) / np.linalg.norm(want) < 5e-3


def test_seeded_golden_vectors_are_reproduced(oracle, seeded):
    """The committed vectors are what the oracle computes today (bit for bit)."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    import helpers
    for name, args in mg.CASES.items():
        case = mg.build_case(oracle, helpers, *args)
        for key, val in case.items():
            assert np.array_equal(np.asarray(val), seeded[f"{name}/{key}"]), (name, key)


def _norm_f64(v, weight, eps, bias=0.0):
    v = v.astype(np.float64)
    inv = 1.0 / np.sqrt((v * v).mean(axis=1, keepdims=True) + eps)
    return v * inv * (bias + weight.astype(np.float64))


def test_rmsnorm_checkers_match_closed_form(oracle, golden):
    """The norm restatements on the upstream test inputs against float64 algebra."""
    c = golden["rmsnorm_f32"]
    x = np.array(c["x"], np.float32).reshape(c["rows"], c["hidden"])
    w = np.array(c["weight"], np.float32)
    assert np.allclose(oracle.rmsnorm(x, w, c["eps"]), _norm_f64(x, w, c["eps"]), atol=1e-6)
    assert np.allclose(oracle.rmsnorm(x, w, c["eps"], 1.0), _norm_f64(x, w, c["eps"], 1.0), atol=1e-6)
    for name, conv in (("fused_add_rmsnorm_f32", lambda a: a), ("fused_add_rmsnorm_bf16", bf16)):
        c = golden[name]
        shape = (c["rows"], c["hidden"])
        x = np.array(c["x"], np.float32).reshape(shape)
        r = np.array(c["residual"], np.float32).reshape(shape)
        w = np.array(c["weight"], np.float32)
        norm, res = oracle.fused_add_rmsnorm(conv(x), conv(r), conv(w), c["eps"])
        assert np.array_equal(res, x + r)            # the inputs are exactly representable
        assert np.allclose(norm, _norm_f64(x + r, w, c["eps"]), atol=1e-6)
