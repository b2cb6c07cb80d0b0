"""GPU parity of the NVFP4 path: quantisers and scale layouts bit-exact against the
CPU oracle, routed experts and the whole layer within the stated output tolerance.
Upstream has no NVFP4 arithmetic, so these outputs are pinned to the oracle only."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, make_moe_inputs, max_abs, rel_l2, to_dev, to_np, zipf_bias

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def ctx(ops):
    return ops.Context()


def test_activation_quantiser_is_bit_exact(ops, ctx, oracle):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((37, 256), dtype=np.float32)
    x[0, :16] = 0.0                       # all-zero block -> scale 0, codes 0
    x[1, :16] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
    x[2] *= 1e-4                          # tiny values: sub-normal block scales
    x[3] *= 300.0
    xb = bf16(x)
    for g in (1.0, 0.37):
        packed, scale = ops.nvfp4_quantize_act(ctx, to_dev(xb), g)
        p_ref, s_ref = oracle.nvfp4_quantize_act(xb, g)
        assert np.array_equal(to_np(scale), s_ref)
        assert np.array_equal(to_np(packed), p_ref)


@pytest.mark.parametrize("gated", [False, True])
def test_weight_quantiser_and_scale_tiling_are_bit_exact(ops, ctx, oracle, gated):
    rng = np.random.default_rng(22)
    e, rows, k = 3, 256, 512
    w = bf16(rng.standard_normal((e, rows, k), dtype=np.float32) * 0.02)
    w[1] = 0  # all-zero expert: global scale 1
    q = ops.nvfp4_quantize_weight(ctx, to_dev(w), gated)
    p_ref, s_ref, st_ref, g_ref = oracle.nvfp4_quantize_weight(w, gated)
    assert np.array_equal(to_np(q.global_scale), g_ref)
    assert np.array_equal(to_np(q.scale_linear), s_ref)
    assert np.array_equal(to_np(q.packed), p_ref)
    assert np.array_equal(to_np(q.scale_tiled), st_ref)
    # re-tiling the declared (linear) layout gives the same tiled buffer
    assert np.array_equal(to_np(ops.nvfp4_tile_scales(ctx, q.scale_linear, gated)), st_ref)


def _check(out, ref):
    assert rel_l2(out, ref) <= 1e-2
    assert max_abs(out, ref) <= 2.0 ** -5 * np.max(np.abs(f32(ref)))


def _quantise_all(ops, ctx, d, shared):
    gu = ops.nvfp4_quantize_weight(ctx, to_dev(d["gate_up"]), True)
    dn = ops.nvfp4_quantize_weight(ctx, to_dev(d["down"]), False)
    sh = None
    if shared:
        sh = (ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_gate_up"]), True),
              ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_down"]), False))
    return gu, dn, sh


def _triple(q):
    return to_np(q.packed), to_np(q.scale_linear), to_np(q.global_scale)


@pytest.mark.parametrize("cfg", [
    dict(t=64, h=256, e=8, k=2, i=256),
    dict(t=200, h=512, e=16, k=4, i=256, local=(4, 8)),
])
def test_declared_abi_execute_matches_oracle(ops, ctx, oracle, cfg):
    """qsfi_moe_execute_nvfp4 with the declared (pre-quantised, linear-scale) layout."""
    t, h, e, k, i = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"]
    off, le = cfg.get("local", (0, e))
    d = make_moe_inputs(31, t, h, e, i)
    d["gate_up"], d["down"] = d["gate_up"][off:off + le], d["down"][off:off + le]
    ids, w = oracle.router_topk(oracle.gemm_bf16(d["hidden"], d["router"], "f32"), k, 0, True, 1.0)
    # the declared ABI has no per-expert scale for the gate_up product, so its weights are
    # quantised against a global scale of 1 (weights scaled up so that block scales stay normal)
    gu_w = bf16(f32(d["gate_up"]) * 8.0)
    dn_w = bf16(f32(d["down"]) * 8.0)
    gup, gus = oracle.nvfp4_quantize_act(gu_w.reshape(-1, h), 1.0)
    dnp, dns = oracle.nvfp4_quantize_act(dn_w.reshape(-1, i), 1.0)
    gup, gus = gup.reshape(le, 2 * i, h // 2), gus.reshape(le, 2 * i, h // 16)
    dnp, dns = dnp.reshape(le, h, i // 2), dns.reshape(le, h, i // 16)
    out_scale = (0.5 + d["rng"].random(le)).astype(np.float32)
    hp, hs = ops.nvfp4_quantize_act(ctx, to_dev(d["hidden"]), 1.0)
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, local_expert_offset=off,
                                              local_num_experts=le, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ops.moe_execute_nvfp4(plan, hp, hs, to_dev(ids), to_dev(w), to_dev(gup), to_dev(gus), to_dev(dnp),
                          to_dev(dns), out, ws, expert_output_scale=to_dev(out_scale))
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    ones = np.ones(le, np.float32)
    ref = oracle.moe_nvfp4(to_np(hp), to_np(hs), ids, w, (gup, gus, ones), (dnp, dns, out_scale),
                           local_offset=off)
    _check(to_np(out), ref)


@pytest.mark.parametrize("cfg", [
    dict(t=64, h=256, e=8, k=2, i=256, s=0),
    dict(t=300, h=512, e=32, k=4, i=256, s=256, bias=True),
    dict(t=128, h=2048, e=64, k=10, i=512, s=512, bias=True),   # layer shape of the prefill workload
])
def test_whole_layer_matches_oracle(ops, ctx, oracle, cfg):
    t, h, e, k, i, s = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"], cfg["s"]
    d = make_moe_inputs(33, t, h, e, i, s)
    bias = zipf_bias(e, d["rng"]) if cfg.get("bias") else None
    gu, dn, sh = _quantise_all(ops, ctx, d, bool(s))
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    logits_t = torch.empty((t, e), dtype=torch.float32, device="cuda")
    shared = None
    if s:
        shared = ops.SharedExpert(sh[0], sh[1], to_dev(d["sh_gate"]), s)
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), gu, dn, out, ws,
                          router_bias=None if bias is None else to_dev(bias), shared=shared,
                          topk_ids=ids_t, topk_weights=w_t, router_logits=logits_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    ids_ref, w_ref = oracle.router_topk(to_np(logits_t), k, 0, True, 1.0, bias)
    assert np.array_equal(to_np(ids_t), ids_ref)
    hp, hs = oracle.nvfp4_quantize_act(d["hidden"], 1.0)
    shared_ref = None
    if s:
        shared_ref = dict(gu=_triple(sh[0]), d=_triple(sh[1]), gate_w=d["sh_gate"])
    ref = oracle.moe_nvfp4(hp, hs, ids_ref, w_ref, _triple(gu), _triple(dn), shared=shared_ref,
                           hidden_bf16=d["hidden"])
    _check(to_np(out), ref)
    # and against the unquantised bf16 chain: NVFP4 is a lossy format, so only a loose bound
    full = oracle.moe_bf16(d["hidden"], ids_ref, w_ref, d["gate_up"], d["down"])
    if s:
        full = oracle.shared_expert_bf16(d["hidden"], d["sh_gate_up"], d["sh_down"], d["sh_gate"], full)
    assert rel_l2(to_np(out), full) <= 0.25


def test_layer_call_replays_from_a_cuda_graph(ops, oracle):
    """The whole-layer call (with its internal side-stream fork for the shared expert) captured
    once in a CUDA graph and replayed on fresh inputs gives the eager result bit for bit."""
    t, h, e, k, i, s = 256, 512, 32, 4, 256, 256
    d = make_moe_inputs(35, t, h, e, i, s)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = ops.Context()          # bound to this (non-default) stream
        gu, dn, sh = _quantise_all(ops, ctx, d, True)
        shared = ops.SharedExpert(sh[0], sh[1], to_dev(d["sh_gate"]), s)
        plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                                  num_experts=e, top_k=k, backend=ops.capi.MOE_BACKEND_NVFP4))
        ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
        x = to_dev(d["hidden"])
        router = to_dev(d["router"])
        out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
        run = lambda: ops.moe_layer_execute(plan, x, router, gu, dn, out, ws, shared=shared)
        for _ in range(2):
            run()
        stream.synchronize()
        eager_first = to_np(out)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        # new tokens in the same buffer: the graph must recompute everything from them
        x.copy_(to_dev(bf16(f32(d["hidden"])[::-1].copy())))
        graph.replay()
        stream.synchronize()
        replayed = to_np(out)
        run()
        stream.synchronize()
        assert ctx.read_device_error() == 0
        assert np.array_equal(replayed, to_np(out))
        assert not np.array_equal(replayed, eager_first)


def test_gate_and_up_rows_with_separate_global_scales(ops, ctx, oracle):
    """Checkpoints that quantise gate_proj and up_proj apart carry one global scale for each;
    the layer takes them as f32 [2 * experts] (routed) and f32 [2] (shared expert)."""
    import dataclasses
    t, h, e, k, i, s = 96, 512, 16, 4, 256, 256
    d = make_moe_inputs(37, t, h, e, i, s)
    gu, dn, sh = _quantise_all(ops, ctx, d, True)
    factor = torch.linspace(0.6, 1.7, e, device="cuda")
    gu2 = dataclasses.replace(gu, global_scale=torch.cat([gu.global_scale, gu.global_scale * factor]))
    sgu2 = dataclasses.replace(sh[0], global_scale=torch.cat([sh[0].global_scale, sh[0].global_scale * 1.3]))
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    shared = ops.SharedExpert(sgu2, sh[1], to_dev(d["sh_gate"]), s)
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), gu2, dn, out, ws, shared=shared,
                          topk_ids=ids_t, topk_weights=w_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    hp, hs = oracle.nvfp4_quantize_act(d["hidden"], 1.0)
    ref = oracle.moe_nvfp4(hp, hs, to_np(ids_t), to_np(w_t), _triple(gu2), _triple(dn),
                           shared=dict(gu=_triple(sgu2), d=_triple(sh[1]), gate_w=d["sh_gate"]),
                           hidden_bf16=d["hidden"])
    _check(to_np(out), ref)
    # the second scale is really applied: the single-scale result differs
    single = oracle.moe_nvfp4(hp, hs, to_np(ids_t), to_np(w_t), _triple(gu), _triple(dn),
                              shared=dict(gu=_triple(sh[0]), d=_triple(sh[1]), gate_w=d["sh_gate"]),
                              hidden_bf16=d["hidden"])
    assert rel_l2(to_np(out), single) > 0.05


@pytest.mark.parametrize("cfg", [
    dict(t=16, h=512, e=64, k=4, i=256, s=256),                 # a few rows per expert, most experts empty
    dict(t=128, h=2048, e=128, k=10, i=512, s=512, bias=True),  # decode batch of the prefill layer's shape
    dict(t=40, h=256, e=4, k=2, i=256, s=0),                    # 80 routes on 4 experts: several 32-row tiles each
])
def test_decode_batches_take_the_swapped_operand_kernel(ops, ctx, oracle, cfg):
    """With at most 16 routes per expert on average the plan pads expert segments to 32 rows and
    the grouped GEMMs run with the weights as the M side of the MMA; same results as the oracle."""
    t, h, e, k, i, s = cfg["t"], cfg["h"], cfg["e"], cfg["k"], cfg["i"], cfg["s"]
    assert t * k <= 16 * e or e == 4
    d = make_moe_inputs(41, t, h, e, i, s)
    bias = zipf_bias(e, d["rng"]) if cfg.get("bias") else None
    gu, dn, sh = _quantise_all(ops, ctx, d, bool(s))
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    shared = ops.SharedExpert(sh[0], sh[1], to_dev(d["sh_gate"]), s) if s else None
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), to_dev(d["router"]), gu, dn, out, ws,
                          router_bias=None if bias is None else to_dev(bias), shared=shared,
                          act_global_scale=0.5, act2_global_scale=0.25, topk_ids=ids_t, topk_weights=w_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    hp, hs = oracle.nvfp4_quantize_act(d["hidden"], 0.5)
    shared_ref = dict(gu=_triple(sh[0]), d=_triple(sh[1]), gate_w=d["sh_gate"]) if s else None
    ref = oracle.moe_nvfp4(hp, hs, to_np(ids_t), to_np(w_t), _triple(gu), _triple(dn), act_global=0.5,
                           act2_global=0.25, shared=shared_ref, hidden_bf16=d["hidden"])
    _check(to_np(out), ref)
