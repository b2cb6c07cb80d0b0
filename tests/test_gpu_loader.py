"""GPU side of the checkpoint loader: synthetic safetensors checkpoints of one MoE layer,
loaded through the pinned staging ring into the layouts the layer call consumes. Loaded
tensors are compared bit for bit with what the files hold (or with the device quantiser
applied to it), and the layer run on the loaded weights is compared with the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import (bf16, f32, make_moe_inputs, max_abs, moe_checkpoint_tensors, rel_l2, to_dev, to_np,
                     write_safetensors)

pytestmark = pytest.mark.gpu
PREFIX = "model.language_model.layers.7.mlp."


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def loader():
    from qs3_b200 import loader as m
    return m


@pytest.fixture(scope="module")
def ctx(ops):
    return ops.Context()


def _checkpoint(tmp_path, loader, ctx, d, **kw):
    tensors, ref = moe_checkpoint_tensors(PREFIX, d, **kw)
    names = list(tensors)
    half = len(names) // 2     # two shards, no index
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half:]})
    return loader.Checkpoint(ctx, str(tmp_path)), ref


@pytest.mark.parametrize("transposed", [False, True])
def test_bf16_checkpoint_loads_bit_exact_and_runs(tmp_path, ops, loader, ctx, oracle, transposed):
    t, h, e, k, i, s = 48, 256, 20, 4, 96, 64          # 20 experts: three staging chunks
    d = make_moe_inputs(61, t, h, e, i, s)
    ck, _ = _checkpoint(tmp_path, loader, ctx, d, nvfp4=False, transposed=transposed)
    dims = dict(hidden=h, inter=i, experts=e, shared_inter=s)
    w = loader.load_moe_layer(ck, PREFIX, **dims)
    assert np.array_equal(to_np(w.router), d["router"])
    assert np.array_equal(to_np(w.gate_up), d["gate_up"])
    assert np.array_equal(to_np(w.down), d["down"])
    assert np.array_equal(to_np(w.shared.gate_up), d["sh_gate_up"])
    assert np.array_equal(to_np(w.shared.down), d["sh_down"])
    assert np.array_equal(to_np(w.shared.gate_weight), d["sh_gate"])
    assert (w.act_global_scale, w.act2_global_scale) == (1.0, 1.0)
    # a rank that owns physical positions 5..15 of a permuted placement
    order = np.random.default_rng(3).permutation(e)
    part = loader.load_moe_layer(ck, PREFIX, local=(5, 11), expert_order=order, **dims)
    assert np.array_equal(to_np(part.router), d["router"][order])
    assert np.array_equal(to_np(part.gate_up), d["gate_up"][order[5:16]])
    assert np.array_equal(to_np(part.down), d["down"][order[5:16]])
    # the loaded layer computes what the oracle computes from the same arrays
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i, num_experts=e,
                                              top_k=k))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), w.router, w.gate_up, w.down, out, ws, shared=w.shared,
                          topk_ids=ids_t, topk_weights=w_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    ref = oracle.moe_bf16(d["hidden"], to_np(ids_t), to_np(w_t), d["gate_up"], d["down"])
    ref = oracle.shared_expert_bf16(d["hidden"], d["sh_gate_up"], d["sh_down"], d["sh_gate"], ref)
    assert rel_l2(to_np(out), ref) <= 1e-2


def test_bf16_checkpoint_quantised_at_load_time(tmp_path, ops, loader, ctx):
    """BF16 file, NVFP4 plan: the loader's staged quantisation equals the device quantiser
    applied to the whole tensors."""
    h, e, i, s = 256, 11, 128, 128
    d = make_moe_inputs(62, 4, h, e, i, s)
    ck, _ = _checkpoint(tmp_path, loader, ctx, d, nvfp4=False, transposed=True)
    # hidden == 2 * intermediate: the shape of gate_up_proj does not tell its layout, the caller does
    w = loader.load_moe_layer(ck, PREFIX, hidden=h, inter=i, experts=e, shared_inter=s,
                              backend=ops.capi.MOE_BACKEND_NVFP4, fused_transposed=True)
    for got, src, gated in [(w.gate_up, d["gate_up"], True), (w.down, d["down"], False),
                            (w.shared.gate_up, d["sh_gate_up"], True), (w.shared.down, d["sh_down"], False)]:
        want = ops.nvfp4_quantize_weight(ctx, to_dev(src), gated)
        assert np.array_equal(to_np(got.packed), to_np(want.packed))
        assert np.array_equal(to_np(got.scale_tiled), to_np(want.scale_tiled))
        assert np.array_equal(to_np(got.global_scale), to_np(want.global_scale))


def _check(out, ref):
    assert rel_l2(out, ref) <= 1e-2
    assert max_abs(out, ref) <= 2.0 ** -5 * np.max(np.abs(f32(ref)))


@pytest.mark.parametrize("shared_nvfp4", [True, False])
def test_nvfp4_checkpoint_loads_and_runs(tmp_path, ops, loader, ctx, oracle, shared_nvfp4):
    t, h, e, k, i, s = 80, 256, 19, 4, 256, 256
    d = make_moe_inputs(63, t, h, e, i, s)
    ck, ref = _checkpoint(tmp_path, loader, ctx, d, nvfp4=True, shared_nvfp4=shared_nvfp4)
    capi = ops.capi
    kw = dict(hidden=h, inter=i, experts=e, shared_inter=s, fmt=capi.CHECKPOINT_EXPERTS_NVFP4_SPLIT,
              backend=capi.MOE_BACKEND_NVFP4)
    w = loader.load_moe_layer(ck, PREFIX, **kw)
    gu_p, gu_s, gu_g = ref["gu"]
    d_p, d_s, d_g = ref["d"]
    assert np.array_equal(to_np(w.router), d["router"])
    assert np.array_equal(to_np(w.gate_up.packed), gu_p)          # gate rows then up rows of every expert
    assert np.array_equal(to_np(w.down.packed), d_p)
    assert np.array_equal(to_np(w.gate_up.global_scale), gu_g.reshape(-1))   # [2, E]: gate scales, up scales
    assert np.array_equal(to_np(w.down.global_scale), d_g)
    # block scales: re-tiling the declared linear layout gives the loaded buffers
    assert np.array_equal(to_np(w.gate_up.scale_tiled), to_np(ops.nvfp4_tile_scales(ctx, to_dev(gu_s), True)))
    assert np.array_equal(to_np(w.down.scale_tiled), to_np(ops.nvfp4_tile_scales(ctx, to_dev(d_s), False)))
    assert w.act_global_scale == pytest.approx(ref["act"], rel=0, abs=0)
    assert w.act2_global_scale == pytest.approx(ref["act2"], rel=0, abs=0)
    if shared_nvfp4:
        sp, ss, sg = ref["sh_gu"]
        assert np.array_equal(to_np(w.shared.gate_up.packed), sp)
        assert np.array_equal(to_np(w.shared.gate_up.global_scale), sg)
        assert np.array_equal(to_np(w.shared.gate_up.scale_tiled), to_np(ops.nvfp4_tile_scales(ctx, to_dev(ss), True)))
        shared_ref = dict(gu=ref["sh_gu"], d=ref["sh_d"], gate_w=d["sh_gate"])
    else:
        q_gu = ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_gate_up"]), True)
        q_d = ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_down"]), False)
        assert np.array_equal(to_np(w.shared.gate_up.packed), to_np(q_gu.packed))
        assert np.array_equal(to_np(w.shared.down.scale_tiled), to_np(q_d.scale_tiled))
        triple = lambda q: (to_np(q.packed), to_np(q.scale_linear), to_np(q.global_scale))
        shared_ref = dict(gu=triple(q_gu), d=triple(q_d), gate_w=d["sh_gate"])
    # a rank holding a slice of a permuted placement gets the matching rows of everything
    order = np.random.default_rng(4).permutation(e)
    part = loader.load_moe_layer(ck, PREFIX, local=(9, 10), expert_order=order, **kw)
    sel = order[9:19]
    assert np.array_equal(to_np(part.gate_up.packed), gu_p[sel])
    assert np.array_equal(to_np(part.gate_up.global_scale), gu_g[:, sel].reshape(-1))
    assert np.array_equal(to_np(part.down.scale_tiled), to_np(ops.nvfp4_tile_scales(ctx, to_dev(d_s[sel]), False)))
    assert part.act_global_scale == w.act_global_scale            # every rank quantises tokens alike

    # the layer on the loaded weights, with the checkpoint's activation scales, against the oracle
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i, num_experts=e,
                                              top_k=k, backend=capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    ids_t = torch.empty((t, k), dtype=torch.int32, device="cuda")
    w_t = torch.empty((t, k), dtype=torch.float32, device="cuda")
    ops.moe_layer_execute(plan, to_dev(d["hidden"]), w.router, w.gate_up, w.down, out, ws, shared=w.shared,
                          act_global_scale=w.act_global_scale, act2_global_scale=w.act2_global_scale,
                          topk_ids=ids_t, topk_weights=w_t)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    hp, hs = oracle.nvfp4_quantize_act(d["hidden"], w.act_global_scale)
    want = oracle.moe_nvfp4(hp, hs, to_np(ids_t), to_np(w_t), ref["gu"], ref["d"], act_global=w.act_global_scale,
                            act2_global=w.act2_global_scale, shared=shared_ref, hidden_bf16=d["hidden"])
    _check(to_np(out), want)
    # NVFP4 is lossy: against the unquantised chain only a loose bound holds
    full = oracle.moe_bf16(d["hidden"], to_np(ids_t), to_np(w_t), d["gate_up"], d["down"])
    full = oracle.shared_expert_bf16(d["hidden"], d["sh_gate_up"], d["sh_down"], d["sh_gate"], full)
    assert rel_l2(to_np(out), full) <= 0.25
