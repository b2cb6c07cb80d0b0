"""GPU parity of the FP8 block-scaled path (e4m3 weights with 128 x 128 f32 block scales,
e4m3 activations with per-token 128-element groups): quantisers bit-exact against the CPU
oracle, routed experts and the whole layer within the stated output tolerance. Upstream
has no FP8 MoE arithmetic, so these outputs are pinned to the oracle only."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, make_moe_inputs, max_abs, rel_l2, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def ctx(ops):
    return ops.Context()


def _check(out, ref):
    assert rel_l2(out, ref) <= 1e-2
    assert max_abs(out, ref) <= 2.0 ** -5 * np.max(np.abs(f32(ref)))


def test_activation_quantiser_is_bit_exact(ops, ctx, oracle):
    rng = np.random.default_rng(41)
    x = rng.standard_normal((37, 384), dtype=np.float32)
    x[0, :128] = 0.0          # all-zero group: floor scale, codes 0
    x[1] *= 1e-5
    x[2] *= 3e4
    x[3, :8] = [448.0, -448.0, 224.0, 0.015625, 0.001953125, -0.0009765625, 1.0, -1.0]
    xb = bf16(x)
    codes, scale = ops.fp8_quantize_act(ctx, to_dev(xb))
    c_ref, s_ref = oracle.fp8_quantize_act(xb)
    assert np.array_equal(to_np(scale), s_ref)
    assert np.array_equal(to_np(codes), c_ref)


def test_weight_quantiser_is_bit_exact(ops, ctx, oracle):
    rng = np.random.default_rng(42)
    e, rows, k = 3, 320, 256   # 320 rows: the last row block is partial
    w = bf16(rng.standard_normal((e, rows, k), dtype=np.float32) * 0.02)
    w[1, :128, :128] = 0
    q = ops.fp8_quantize_weight(ctx, to_dev(w))
    c_ref, s_ref = oracle.fp8_quantize_weight(w)
    assert np.array_equal(to_np(q.scale), s_ref)
    assert np.array_equal(to_np(q.codes), c_ref)


def _plan(ops, ctx, t, h, i, e, k, off=0, le=None):
    return ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, local_expert_offset=off,
                                              local_num_experts=le,
                                              backend=ops.capi.MOE_BACKEND_FP8_BLOCKSCALE))


@pytest.mark.parametrize("cfg", [
    dict(t=16, h=256, e=8, k=2, i=128),                       # a few rows per expert, 16-row token tiles
    dict(t=40, h=512, e=4, k=2, i=256),                       # 20 rows per expert: two 16-row tiles each
    dict(t=200, h=512, e=4, k=2, i=256),                      # 100 rows per expert: 32-row token tiles
    dict(t=96, h=384, e=16, k=4, i=128, local=(4, 8)),        # partial local expert range
    dict(t=64, h=2048, e=128, k=8, i=768),                    # decode configuration (Qwen3-30B-A3B shape)
])
def test_execute_fp8_matches_oracle(ops, ctx, oracle, cfg):
    t, h, e, k, i = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"]
    off, le = cfg.get("local", (0, e))
    d = make_moe_inputs(43, t, h, e, i)
    ids, w = oracle.router_topk(oracle.gemm_bf16(d["hidden"], d["router"], "f32"), k, 0, True, 1.0)
    gu = ops.fp8_quantize_weight(ctx, to_dev(d["gate_up"][off:off + le]))
    dn = ops.fp8_quantize_weight(ctx, to_dev(d["down"][off:off + le]))
    hc, hs = ops.fp8_quantize_act(ctx, to_dev(d["hidden"]))
    plan = _plan(ops, ctx, t, h, i, e, k, off, le)
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ops.moe_execute_fp8(plan, hc, hs, to_dev(ids), to_dev(w), gu, dn, out, ws)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    ref = oracle.moe_fp8(to_np(hc), to_np(hs), ids, w, (to_np(gu.codes), to_np(gu.scale)),
                         (to_np(dn.codes), to_np(dn.scale)), local_offset=off)
    _check(to_np(out), ref)
    # against the unquantised bf16 chain: FP8 is lossy, so only a loose bound
    full = oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"][off:off + le], d["down"][off:off + le], off)
    assert rel_l2(to_np(out), full) <= 0.1


def test_execute_fp8_is_deterministic_and_linear_in_routing_weight(ops, ctx, oracle):
    """Size-independent properties: two runs agree bit for bit, and doubling every routing
    weight doubles the output (up to the final bf16 rounding)."""
    t, h, e, k, i = 64, 512, 32, 4, 256
    d = make_moe_inputs(44, t, h, e, i)
    ids, w = oracle.router_topk(oracle.gemm_bf16(d["hidden"], d["router"], "f32"), k, 0, True, 1.0)
    gu = ops.fp8_quantize_weight(ctx, to_dev(d["gate_up"]))
    dn = ops.fp8_quantize_weight(ctx, to_dev(d["down"]))
    hc, hs = ops.fp8_quantize_act(ctx, to_dev(d["hidden"]))
    plan = _plan(ops, ctx, t, h, i, e, k)
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    outs = []
    for scale in (1.0, 1.0, 2.0):
        out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
        ops.moe_execute_fp8(plan, hc, hs, to_dev(ids), to_dev(w * np.float32(scale)), gu, dn, out, ws)
        torch.cuda.synchronize()
        outs.append(to_np(out))
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(f32(outs[2]), 2.0 * f32(outs[0]))


@pytest.mark.parametrize("cfg", [
    dict(t=32, h=256, e=8, k=2, i=128),
    dict(t=64, h=2048, e=128, k=8, i=768),   # decode configuration
])
def test_whole_layer_fp8_matches_oracle(ops, ctx, oracle, cfg):
    t, h, e, k, i = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"]
    d = make_moe_inputs(45, t, h, e, i)
    gu = ops.fp8_quantize_weight(ctx, to_dev(d["gate_up"]))
    dn = ops.fp8_quantize_weight(ctx, to_dev(d["down"]))
    plan = _plan(ops, ctx, t, h, i, e, k)
    ws = torch.zeros(plan.layer_workspace_size(t, 0), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    logits_t = torch.empty((t, e), dtype=torch.float32, device="cuda")
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), gu, dn, out, ws,
                          topk_ids=ids_t, topk_weights=w_t, router_logits=logits_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    ids_ref, w_ref = oracle.router_topk(to_np(logits_t), k, 0, True, 1.0)
    assert np.array_equal(to_np(ids_t), ids_ref)
    hc, hs = oracle.fp8_quantize_act(d["hidden"])
    ref = oracle.moe_fp8(hc, hs, ids_ref, w_ref, (to_np(gu.codes), to_np(gu.scale)),
                         (to_np(dn.codes), to_np(dn.scale)))
    _check(to_np(out), ref)


def test_fp8_plan_validation(ops, ctx):
    with pytest.raises(ops.Qs3Error, match="divisible by 128"):
        _plan(ops, ctx, 8, 192, 128, 4, 2)
    with pytest.raises(ops.Qs3Error, match="up to 4096"):
        _plan(ops, ctx, 8, 8192, 128, 4, 2)
