"""GPU parity of the bf16 MoE path (qsfi_moe_execute_bf16 and the whole-layer call)
against the strict-chain CPU oracle and the upstream known-answer cases."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, make_moe_inputs, max_abs, moe_case_arrays, rel_l2, to_dev, to_np

pytestmark = pytest.mark.gpu

SENTINEL = 0xA5A5  # upstream test.cu:25


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


def _execute(ops, hidden, ids, w, gate_up, down, experts, local=(0, None), guard_rows=3):
    t, h = hidden.shape
    le = gate_up.shape[0]
    i = gate_up.shape[1] // 2
    ctx = ops.Context()
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=experts, top_k=ids.shape[1],
                                              local_expert_offset=local[0], local_num_experts=le))
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    # output rows are followed by sentinel rows that must survive the call
    buf = torch.from_numpy(np.full((t + guard_rows, h), SENTINEL, np.uint16)).view(torch.bfloat16).cuda()
    out = buf[:t]
    ops.moe_execute_bf16(plan, to_dev(hidden), to_dev(ids), to_dev(w), to_dev(gate_up), to_dev(down), out, ws)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    got = to_np(buf)
    assert np.all(got[t:] == SENTINEL), "wrote past the output tensor"
    return got[:t], plan, ws


@pytest.mark.parametrize("name", ["moe_staged_grouped_gemm", "moe_top2_weighted_accumulation"])
def test_upstream_known_answers(ops, golden, name):
    case = golden[name]
    hidden, ids, w, gate_up, down, expected = moe_case_arrays(case)
    out, _, _ = _execute(ops, hidden, ids, w, gate_up, down, case["experts"])
    got = f32(out)
    assert np.max(np.abs(got - expected)) <= case["tolerance"]
    assert np.all(got[expected == 0.0] == 0.0)


def _check(out, ref):
    assert rel_l2(out, ref) <= 1e-2  # the stated bf16 output tolerance
    scale = np.max(np.abs(f32(ref)))
    assert max_abs(out, ref) <= 2.0 ** -6 * scale


@pytest.mark.parametrize("cfg", [
    dict(t=16, h=256, e=8, k=2, i=128),      # the tiny bf16 configuration
    dict(t=5, h=8, e=3, k=2, i=16),          # reduction shorter than a tile: CUDA-core kernel
    dict(t=77, h=72, e=5, k=3, i=40),        # ragged k and n tails on the tensor-core kernel
    dict(t=300, h=512, e=16, k=4, i=192),    # several row tiles per expert
    dict(t=64, h=1024, e=64, k=8, i=256, hot=True),
])
def test_matches_oracle(ops, oracle, cfg):
    t, h, e, k, i = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"]
    d = make_moe_inputs(1, t, h, e, i)
    logits = oracle.gemm_bf16(d["hidden"], d["router"], "f32")
    if cfg.get("hot"):
        logits[:, 3] += 10.0  # every token picks expert 3: one long segment, many empty ones
    ids, w = oracle.router_topk(logits, k, 0, True, 1.0)
    out, plan, ws = _execute(ops, d["hidden"], ids, w, d["gate_up"], d["down"], e)
    ref = oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"], d["down"])
    _check(out, ref)
    tables = [to_np(x) for x in plan.routing_tables(ws, t)]
    for g, r in zip(tables, oracle.route_sort(ids, w, 0, e)):
        assert np.array_equal(g, r)


def test_expert_parallel_partials_sum_to_the_full_result(ops, oracle):
    t, h, e, k, i = 48, 256, 8, 2, 128
    d = make_moe_inputs(2, t, h, e, i)
    ids, w = oracle.router_topk(oracle.gemm_bf16(d["hidden"], d["router"], "f32"), k, 0, True, 1.0)
    total = np.zeros((t, h), np.float64)
    for rank in range(2):
        lo = rank * 4
        out, _, _ = _execute(ops, d["hidden"], ids, w, d["gate_up"][lo:lo + 4], d["down"][lo:lo + 4], e,
                             local=(lo, 4))
        ref = oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"][lo:lo + 4], d["down"][lo:lo + 4], local_offset=lo)
        _check(out, ref)
        total += f32(out)
    full = f32(oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"], d["down"])).astype(np.float64)
    assert np.linalg.norm(total - full) <= 1e-2 * np.linalg.norm(full)


def test_runtime_validation_messages(ops):
    ctx = ops.Context()
    ctx.validate_target()  # compute capability 10.0
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=4, hidden_size=64, intermediate_size=64,
                                              num_experts=2, top_k=1))
    z = lambda *s, dt=torch.bfloat16: torch.zeros(s, dtype=dt, device="cuda")
    ws = z(plan.workspace_size(4), dt=torch.uint8)
    with pytest.raises(ops.Qs3Error) as e:
        ops.moe_execute_bf16(plan, z(4, 64), z(4, 1, dt=torch.int32), z(4, 1, dt=torch.float32),
                             z(2, 128, 64), z(2, 64, 64), z(4, 64), ws[:256])
    assert e.value.status == 1 and "workspace is too small" in e.value.message
    with pytest.raises(ops.Qs3Error) as e:
        ops.moe_execute_bf16(plan, z(4, 64), z(4, 1, dt=torch.int32), z(4, 1, dt=torch.float32),
                             z(2, 128, 64), z(2, 64, 32), z(4, 64), ws)
    assert "expert weight shape mismatch" in e.value.message


@pytest.mark.parametrize("cfg", [
    dict(t=16, h=256, e=8, k=2, i=128, s=0),
    dict(t=130, h=512, e=32, k=4, i=128, s=192, bias=True),
])
def test_whole_layer_matches_oracle(ops, oracle, cfg):
    """Router logits -> top-k -> experts -> shared expert -> combine in one call."""
    t, h, e, k, i, s = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"], cfg["s"]
    d = make_moe_inputs(4, t, h, e, i, s)
    bias = None
    if cfg.get("bias"):
        from helpers import zipf_bias
        bias = zipf_bias(e, d["rng"])
    ctx = ops.Context()
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    logits_t = torch.empty((t, e), dtype=torch.float32, device="cuda")
    shared = None
    if s:
        shared = ops.SharedExpert(to_dev(d["sh_gate_up"]), to_dev(d["sh_down"]), to_dev(d["sh_gate"]), s)
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), to_dev(d["gate_up"]),
                          to_dev(d["down"]), out, ws, router_bias=None if bias is None else to_dev(bias),
                          shared=shared, topk_ids=ids_t, topk_weights=w_t, router_logits=logits_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    logits = to_np(logits_t)
    ref_logits = oracle.gemm_bf16(d["hidden"], d["router"], "f32")
    assert np.allclose(logits, ref_logits, atol=1e-5, rtol=1e-5)
    # routing is bit-exact on identical logits
    ids_ref, w_ref = oracle.router_topk(logits, k, 0, True, 1.0, bias)
    assert np.array_equal(to_np(ids_t), ids_ref)
    assert np.allclose(to_np(w_t), w_ref, atol=1e-5, rtol=0)
    ref = oracle.moe_bf16(d["hidden"], ids_ref, w_ref, d["gate_up"], d["down"])
    if s:
        ref = oracle.shared_expert_bf16(d["hidden"], d["sh_gate_up"], d["sh_down"], d["sh_gate"], ref)
    _check(to_np(out), ref)


@pytest.mark.parametrize("name,shape", [("tiny_bf16", (0, 16, 256, 8, 2, 128)),
                                        ("small_bf16", (1, 48, 128, 16, 4, 64))])
def test_committed_seeded_vectors(ops, seeded, name, shape):
    """Whole bf16 layer against the committed fixtures: expert ids, counts, indptr and the
    permutation bit-exact, output rel-L2 <= 1e-2 (the tiny case is the CPU-runnable
    configuration of the benchmark list: 16 tokens, 8 experts, top-2, seed 0)."""
    seed, t, h, e, k, i = shape
    d = make_moe_inputs(seed, t, h, e, i)
    ctx = ops.Context()
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k))
    ws = torch.zeros(plan.layer_workspace_size(t, 0), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), to_dev(d["gate_up"]),
                          to_dev(d["down"]), out, ws, topk_ids=ids_t, topk_weights=w_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    assert np.array_equal(to_np(ids_t), seeded[f"{name}/ids"])
    assert np.allclose(to_np(w_t), seeded[f"{name}/weights"], atol=1e-5, rtol=0)
    counts, indptr, route_rows, row_tokens, _ = (to_np(x) for x in plan.routing_tables(ws, t))
    assert np.array_equal(counts, seeded[f"{name}/counts"])
    assert np.array_equal(indptr, seeded[f"{name}/indptr"])
    assert np.array_equal(route_rows, seeded[f"{name}/route_rows"])
    assert np.array_equal(row_tokens, seeded[f"{name}/row_tokens"])
    assert rel_l2(to_np(out), seeded[f"{name}/out"]) <= 1e-2
    assert max_abs(to_np(out), seeded[f"{name}/out"]) <= 2.0 ** -6 * np.max(np.abs(f32(seeded[f"{name}/out"])))
