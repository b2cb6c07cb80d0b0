"""A/B against the reference's own GPU code: `qsfi_moe_execute_bf16` and `qscu_router_topk` compiled from
the reference sources (oracle/reference_gpu.py) run on the same seeded inputs as this library.

Upstream's tests pin its BF16 MoE path at two tokens only (test.cu:1455-1703); this compares the two
implementations at the tiny benchmark configuration (16 tokens, 8 experts, top-2) and at a mid-size
shape. Counts and indptr must be equal, every expert's segment must hold the same SET of routes (the
reference places routes inside a segment in atomicAdd order, qsfi_moe.cu:378-382, so the order is not
comparable), every dense row must belong to the token both sides say, and the outputs must agree
within 2^-6 * max|out| (two bf16 GEMM chains with different f32 summation orders)."""
import numpy as np
import pytest
import torch

from helpers import f32, make_moe_inputs, rel_l2, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import reference_gpu
    if not reference_gpu.available():
        pytest.skip("oracle/_ref/libqs3ref.so was not built (the reference tree is needed for that)")
    return reference_gpu, reference_gpu.load()


@pytest.mark.parametrize("shape", [(0, 16, 256, 8, 2, 128), (2, 256, 512, 32, 4, 256), (3, 700, 1024, 16, 8, 512)])
def test_bf16_moe_matches_the_reference_binary(ref, oracle, shape):
    from qs3_b200 import ops
    reference_gpu, ref_lib = ref
    seed, t, h, e, k, i = shape
    d = make_moe_inputs(seed, t, h, e, i)
    ids, w = oracle.router_topk(oracle.gemm_bf16(d["hidden"], d["router"], "f32"), k, 0, True, 1.0)
    outs, tables = {}, {}
    for name, lib in (("ours", None), ("reference", ref_lib)):
        ctx = ops.Context(lib=lib)
        plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                                  num_experts=e, top_k=k))
        ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
        out = torch.zeros((t, h), dtype=torch.bfloat16, device="cuda")
        ops.moe_execute_bf16(plan, to_dev(d["hidden"]), to_dev(ids), to_dev(w), to_dev(d["gate_up"]),
                             to_dev(d["down"]), out, ws)
        torch.cuda.synchronize()
        outs[name] = to_np(out)
        if lib is None:
            tables[name] = [to_np(x) for x in plan.routing_tables(ws, t)[:4]]
        else:
            tables[name] = reference_gpu.workspace_tables(ws, t, k, e)
    (c1, p1, rr1, rt1), (c2, p2, rr2, rt2) = tables["ours"], tables["reference"]
    assert np.array_equal(c1, c2) and np.array_equal(p1, p2)
    flat = ids.ravel()
    for ex in range(e):
        seg = slice(p1[ex], p1[ex + 1])
        routes1 = np.sort(np.nonzero((rr1 >= seg.start) & (rr1 < seg.stop))[0])
        routes2 = np.sort(np.nonzero((rr2 >= seg.start) & (rr2 < seg.stop))[0])
        assert np.array_equal(routes1, routes2) and np.all(flat[routes1] == ex)
    assert np.array_equal(rt1[rr1], np.arange(t * k) // k) and np.array_equal(rt2[rr2], np.arange(t * k) // k)
    a, b = f32(outs["ours"]).astype(np.float64), f32(outs["reference"]).astype(np.float64)
    assert np.max(np.abs(a - b)) <= 2.0 ** -6 * np.max(np.abs(b))
    assert rel_l2(outs["ours"], outs["reference"]) <= 1e-2
    # and both sit where the CPU oracle says
    want = oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"], d["down"])
    assert rel_l2(outs["reference"], want) <= 1e-2 and rel_l2(outs["ours"], want) <= 1e-2


def test_router_matches_the_reference_binary(ref, oracle):
    from qs3_b200 import ops
    _, ref_lib = ref
    rng = np.random.default_rng(8)
    t, e, k = 300, 512, 10
    logits = rng.standard_normal((t, e), dtype=np.float32)
    logits[5, 7] = logits[5, 300] = logits[5, 2] = 3.5          # ties: lowest id first
    logits[9] = np.round(logits[9] * 4) / 4                      # many equal values
    res = {}
    for name, lib in (("ours", None), ("reference", ref_lib)):
        ids = torch.empty((t, k), dtype=torch.int32, device="cuda")
        wts = torch.empty((t, k), dtype=torch.float32, device="cuda")
        ops.router_topk(to_dev(logits), ids, wts, lib=lib)
        torch.cuda.synchronize()
        res[name] = (to_np(ids), to_np(wts))
    assert np.array_equal(res["ours"][0], res["reference"][0])
    assert np.allclose(res["ours"][1], res["reference"][1], atol=1e-5, rtol=0)
    ids_o, w_o = oracle.router_topk(logits, k, 0, True, 1.0)
    assert np.array_equal(res["reference"][0], ids_o) and np.allclose(res["reference"][1], w_o, atol=1e-5, rtol=0)
