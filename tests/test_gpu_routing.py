"""GPU parity of the router, the route permutation and the element-wise helpers,
through the C ABI, against the CPU oracle and the upstream known-answer cases."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, parse_floats, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


def _run_router(ops, logits_np, top_k, score, renorm, scale, as_bf16=False):
    t, e = logits_np.shape
    logits = to_dev(bf16(logits_np)) if as_bf16 else to_dev(logits_np.astype(np.float32))
    ids = torch.full((t, top_k), -7, dtype=torch.int32, device="cuda")
    w = torch.full((t, top_k), -7.0, dtype=torch.float32, device="cuda")
    ops.router_topk(logits, ids, w, score=score, renormalize=renorm, routed_scaling_factor=scale)
    torch.cuda.synchronize()
    return to_np(ids), to_np(w)


@pytest.mark.parametrize("name", ["router_softmax_ties", "router_sigmoid_bf16", "router_nonfinite"])
def test_router_known_answers(ops, oracle, golden, name):
    case = golden[name]
    logits = parse_floats(case["logits"]).reshape(case["num_tokens"], case["num_experts"])
    as_bf16 = name == "router_sigmoid_bf16"
    ids, w = _run_router(ops, logits, case["top_k"], case["score"], bool(case["renormalize"]),
                         case["scale"], as_bf16)
    assert ids.tolist() == case["expected_ids"]
    ref_logits = f32(bf16(logits)) if as_bf16 else logits
    _, w_ref = oracle.router_topk(ref_logits, case["top_k"], case["score"], bool(case["renormalize"]),
                                  case["scale"])
    assert np.all(np.isfinite(w))
    assert np.allclose(w, w_ref, atol=case["weight_tolerance"], rtol=0)
    if "expected_weights" in case:
        assert np.allclose(w, case["expected_weights"], atol=case["weight_tolerance"], rtol=0)


@pytest.mark.parametrize("shape", [(16, 8, 2), (64, 128, 8), (257, 512, 10), (33, 4096, 16), (5, 6, 3),
                                   (1, 1, 1), (1000, 256, 8)])
@pytest.mark.parametrize("score", [0, 1])
def test_router_matches_oracle(ops, oracle, shape, score):
    t, e, k = shape
    rng = np.random.default_rng(1000 * t + e + score)
    logits = rng.standard_normal((t, e), dtype=np.float32) * 1.5
    if score == 1:
        # sigmoid scores saturate and the device uses a fast exp: keep distinct logits
        # far enough apart that score ordering equals logit ordering on both sides
        logits = np.clip(np.round(logits * 4) / 4, -6, 6).astype(np.float32)
    else:
        logits[: t // 2] = np.round(logits[: t // 2] * 2) / 2  # exact ties in half of the rows
    for renorm, scale in ((True, 1.0), (False, 2.5)):
        ids, w = _run_router(ops, logits, k, score, renorm, scale)
        ids_ref, w_ref = oracle.router_topk(logits, k, score, renorm, scale)
        assert np.array_equal(ids, ids_ref)
        assert np.allclose(w, w_ref, atol=1e-5 * scale, rtol=0)
    # bf16 logits take the same path after widening
    lb = f32(bf16(logits))
    ids, w = _run_router(ops, logits, k, score, True, 1.0, as_bf16=True)
    ids_ref, w_ref = oracle.router_topk(lb, k, score, True, 1.0)
    assert np.array_equal(ids, ids_ref)
    assert np.allclose(w, w_ref, atol=1e-5, rtol=0)


def test_router_nan_rows_and_unfilled_slots(ops, oracle):
    logits = np.array([[np.nan, -np.inf, np.nan, 1.0],
                       [np.nan, np.nan, np.nan, np.nan],
                       [np.inf, 0.0, np.inf, -1.0]], np.float32)
    for score in (0, 1):
        ids, w = _run_router(ops, logits, 3, score, True, 1.0)
        ids_ref, w_ref = oracle.router_topk(logits, 3, score, True, 1.0)
        assert np.array_equal(ids, ids_ref)
        assert np.array_equal(np.isnan(w), np.isnan(w_ref))
        m = ~np.isnan(w_ref)
        assert np.allclose(w[m], w_ref[m], atol=1e-5, rtol=0)


def _route_tables(ops, ids_np, w_np, experts, local_offset, local_experts):
    """Run a tiny bf16 MoE (H = I = 8, CUDA-core GEMM) only to obtain the routing tables."""
    t, k = ids_np.shape
    h = i = 8
    ctx = ops.Context()
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=experts, top_k=k,
                                              local_expert_offset=local_offset,
                                              local_num_experts=local_experts))
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    hidden = torch.zeros((t, h), dtype=torch.bfloat16, device="cuda")
    gu = torch.zeros((local_experts, 2 * i, h), dtype=torch.bfloat16, device="cuda")
    dn = torch.zeros((local_experts, h, i), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ops.moe_execute_bf16(plan, hidden, to_dev(ids_np), to_dev(w_np), gu, dn, out, ws)
    tables = [to_np(x) for x in plan.routing_tables(ws, t)]
    assert ctx.read_device_error() == 0
    return tables


@pytest.mark.parametrize("case", [
    dict(t=16, k=2, e=8), dict(t=1, k=1, e=1), dict(t=37, k=4, e=11), dict(t=513, k=10, e=512),
    dict(t=2049, k=8, e=128), dict(t=300, k=3, e=4096, skew=True), dict(t=64, k=2, e=16, one_expert=True),
    dict(t=200, k=6, e=32, local=(8, 8)), dict(t=200, k=6, e=32, local=(24, 8)),
])
def test_route_permutation_is_bit_exact(ops, oracle, case):
    t, k, e = case["t"], case["k"], case["e"]
    rng = np.random.default_rng(7 * t + e)
    if case.get("one_expert"):
        ids = np.full((t, k), 5, np.int32)
    elif case.get("skew"):
        ids = np.minimum((rng.pareto(0.7, size=(t, k)) * 3).astype(np.int64), e - 1).astype(np.int32)
    else:
        ids = rng.integers(0, e, size=(t, k), dtype=np.int32)
    ids[0, :] = ids[0, 0]  # duplicate routes inside one token (upstream test.cu:1586)
    w = rng.random((t, k), dtype=np.float32)
    off, le = case.get("local", (0, e))
    got = _route_tables(ops, ids, w, e, off, le)
    want = oracle.route_sort(ids, w, off, le)
    for name, g, r in zip(("counts", "indptr", "route_rows", "row_tokens", "row_scales"), got, want):
        assert np.array_equal(g, r), name


def test_silu_and_mul(ops, oracle, golden):
    case = golden["silu_and_mul"]
    gate = bf16(case["gate"]).reshape(case["tokens"], case["intermediate"])
    up = bf16(case["up"]).reshape(case["tokens"], case["intermediate"])
    out = torch.full(gate.shape, 12345.0, dtype=torch.bfloat16, device="cuda")
    ops.silu_and_mul_bf16(to_dev(gate), to_dev(up), out)
    g, u = f32(gate).astype(np.float64), f32(up).astype(np.float64)
    assert np.max(np.abs(f32(to_np(out)) - g / (1 + np.exp(-g)) * u)) <= case["tolerance"]
    # larger, vectorised shape against the oracle: at most one bf16 step apart (fast exp on device)
    rng = np.random.default_rng(11)
    gate = bf16(rng.standard_normal((67, 512), dtype=np.float32) * 3)
    up = bf16(rng.standard_normal((67, 512), dtype=np.float32))
    out = torch.empty((67, 512), dtype=torch.bfloat16, device="cuda")
    ops.silu_and_mul_bf16(to_dev(gate), to_dev(up), out)
    ref = f32(oracle.silu_and_mul_bf16(gate, up))
    got = f32(to_np(out))
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30)


def test_shared_expert_gate_add(ops, oracle, golden):
    case = golden["shared_expert_gate_add"]
    rows, hidden = case["rows"], case["hidden"]
    shared = bf16(case["shared"]).reshape(rows, hidden)
    out0 = bf16(case["out"]).reshape(rows, hidden)
    for gate_t in (to_dev(np.array(case["gate"], np.float32).reshape(rows, 1)),
                   to_dev(bf16(case["gate"]).reshape(rows, 1))):
        out = to_dev(out0)
        ops.shared_expert_gate_add_bf16(gate_t, to_dev(shared), out)
        ref = f32(oracle.shared_gate_add_bf16(np.array(case["gate"], np.float32), shared, out0))
        assert np.max(np.abs(f32(to_np(out)) - ref)) <= case["tolerance"]
