"""GPU parity of the RMSNorm neighbours of the MoE block (qsfi_rmsnorm,
qsfi_fused_add_rmsnorm and the variant that also emits NVFP4 codes) against the restated
upstream CPU checkers, on the upstream test vectors and on seeded rows, with the upstream
tolerances (f32: 2e-5 / 1e-5, bf16: 0.018 norm / 0.012 residual)."""
import numpy as np
import pytest
import torch

from helpers import bf16, f32, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def ctx(ops):
    return ops.Context()


def _as_f32(a):
    return f32(a) if a.dtype == np.uint16 else a


@pytest.mark.parametrize("name", ["fused_add_rmsnorm_f32", "fused_add_rmsnorm_bf16"])
def test_upstream_fused_add_vectors(ops, ctx, oracle, golden, name):
    c = golden[name]
    conv = bf16 if name.endswith("bf16") else (lambda a: a)
    shape = (c["rows"], c["hidden"])
    x = conv(np.array(c["x"], np.float32).reshape(shape))
    r = conv(np.array(c["residual"], np.float32).reshape(shape))
    w = conv(np.array(c["weight"], np.float32))
    want_norm, want_res = oracle.fused_add_rmsnorm(x, r, w, c["eps"])
    dx, dr = to_dev(x), to_dev(r)
    ops.fused_add_rmsnorm(ctx, dx, dr, to_dev(w), c["eps"])
    torch.cuda.synchronize()
    assert np.max(np.abs(_as_f32(to_np(dx)) - want_norm)) <= c["abs_tol_norm"]
    assert np.max(np.abs(_as_f32(to_np(dr)) - want_res)) <= c["abs_tol_residual"]


def test_upstream_rmsnorm_vector(ops, ctx, oracle, golden):
    c = golden["rmsnorm_f32"]
    x = np.array(c["x"], np.float32).reshape(c["rows"], c["hidden"])
    w = np.array(c["weight"], np.float32)
    for bias in (0.0, 1.0):
        out = torch.empty((c["rows"], c["hidden"]), dtype=torch.float32, device="cuda")
        ops.rmsnorm(ctx, to_dev(x), to_dev(w), out, c["eps"], bias)
        torch.cuda.synchronize()
        assert np.max(np.abs(to_np(out) - oracle.rmsnorm(x, w, c["eps"], bias))) <= c["abs_tol"]


@pytest.mark.parametrize("rows,hidden,dtype", [(5, 2048, "bf16"), (3, 2048, "f32"), (7, 200, "bf16"),
                                               (2, 12, "f32"), (3, 13, "bf16"), (4, 9000, "bf16"),
                                               (33, 4096, "bf16")])
def test_seeded_rows_match_checker(ops, ctx, oracle, rows, hidden, dtype):
    rng = np.random.default_rng(rows * 31 + hidden)
    conv = bf16 if dtype == "bf16" else (lambda a: a.astype(np.float32))
    x = conv(rng.standard_normal((rows, hidden), dtype=np.float32))
    r = conv(rng.standard_normal((rows, hidden), dtype=np.float32) * 2.0)
    w = conv(1.0 + 0.1 * rng.standard_normal(hidden, dtype=np.float32))
    tol_n, tol_r = (0.06, 0.04) if dtype == "bf16" else (5e-5, 1e-5)  # bf16: half an ulp at |v| < 8
    want_norm, want_res = oracle.fused_add_rmsnorm(x, r, w, 1e-6)
    dx, dr = to_dev(x), to_dev(r)
    ops.fused_add_rmsnorm(ctx, dx, dr, to_dev(w), 1e-6)
    torch.cuda.synchronize()
    assert np.max(np.abs(_as_f32(to_np(dx)) - want_norm)) <= tol_n
    assert np.max(np.abs(_as_f32(to_np(dr)) - want_res)) <= tol_r
    out = torch.empty_like(to_dev(x))
    ops.rmsnorm(ctx, to_dev(x), to_dev(w), out, 1e-6, 1.0)
    torch.cuda.synchronize()
    assert np.max(np.abs(_as_f32(to_np(out)) - oracle.rmsnorm(x, w, 1e-6, 1.0))) <= tol_n


def test_strided_rows(ops, ctx, oracle):
    """Rows with a pitch larger than hidden_size (stride[0] >= shape[1] is legal upstream)."""
    rng = np.random.default_rng(9)
    rows, hidden, pitch = 6, 256, 320
    x = bf16(rng.standard_normal((rows, hidden), dtype=np.float32))
    r = bf16(rng.standard_normal((rows, hidden), dtype=np.float32))
    w = bf16(rng.standard_normal(hidden, dtype=np.float32))
    bx = torch.zeros((rows, pitch), dtype=torch.bfloat16, device="cuda")
    br = torch.zeros((rows, pitch), dtype=torch.bfloat16, device="cuda")
    bx[:, :hidden] = to_dev(x)
    br[:, :hidden] = to_dev(r)
    ops.fused_add_rmsnorm(ctx, bx[:, :hidden], br[:, :hidden], to_dev(w), 1e-6)
    torch.cuda.synchronize()
    want_norm, want_res = oracle.fused_add_rmsnorm(x, r, w, 1e-6)
    assert np.max(np.abs(f32(to_np(bx[:, :hidden].contiguous())) - want_norm)) <= 0.06
    assert np.max(np.abs(f32(to_np(br[:, :hidden].contiguous())) - want_res)) <= 0.04
    assert not to_np(bx[:, hidden:].contiguous()).any()       # the padding columns stay untouched


@pytest.mark.parametrize("rows,hidden", [(16, 2048), (130, 512), (3, 64)])
def test_nvfp4_variant_equals_norm_then_quantise(ops, ctx, oracle, rows, hidden):
    rng = np.random.default_rng(rows + hidden)
    x = bf16(rng.standard_normal((rows, hidden), dtype=np.float32))
    r = bf16(rng.standard_normal((rows, hidden), dtype=np.float32))
    w = bf16(1.0 + 0.1 * rng.standard_normal(hidden, dtype=np.float32))
    # unfused: norm, then the stand-alone activation quantiser on the stored bf16 rows
    ax, ar = to_dev(x), to_dev(r)
    ops.fused_add_rmsnorm(ctx, ax, ar, to_dev(w), 1e-6)
    p_ref, s_ref = oracle.nvfp4_quantize_act(to_np(ax), 0.5)
    # fused
    bx, br = to_dev(x), to_dev(r)
    packed, tiled = ops.fused_add_rmsnorm_nvfp4(ctx, bx, br, to_dev(w), 1e-6, 0.5)
    torch.cuda.synchronize()
    assert np.array_equal(to_np(bx), to_np(ax)) and np.array_equal(to_np(br), to_np(ar))
    assert np.array_equal(to_np(packed), p_ref)
    idx = oracle.tiled_scale_index(rows, hidden)
    assert np.array_equal(to_np(tiled)[idx], s_ref)


def test_validation_messages(ops, ctx):
    x = torch.zeros((2, 8), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.Qs3Error, match="eps must be finite"):
        ops.fused_add_rmsnorm(ctx, x, x.clone(), w, 0.0)
    with pytest.raises(ops.Qs3Error, match="residual_inout shape must match x"):
        ops.fused_add_rmsnorm(ctx, x, torch.zeros((3, 8), dtype=torch.bfloat16, device="cuda"), w, 1e-6)
    with pytest.raises(ops.Qs3Error, match="dtype does not match"):
        ops.fused_add_rmsnorm(ctx, x, x.clone(), w.float(), 1e-6)
    with pytest.raises(ops.Qs3Error, match="supports only bf16/f32"):
        ops.rmsnorm(ctx, x.to(torch.float16), w.to(torch.float16), x.to(torch.float16), 1e-6)
    with pytest.raises(ops.Qs3Error, match="weight_bias must be 0.0 or 1.0"):
        ops.rmsnorm(ctx, x, w, x.clone(), 1e-6, 0.5)


def test_layer_takes_the_tokens_the_norm_quantised(ops, ctx, oracle):
    """Pre-MoE norm that hands its NVFP4 codes to the layer call == norm, then the layer
    quantising for itself (bit for bit), with and without a shared expert."""
    from helpers import make_moe_inputs
    t, h, e, k, i, s = 200, 512, 16, 4, 256, 256
    d = make_moe_inputs(77, t, h, e, i, s)
    rng = d["rng"]
    resid = bf16(rng.standard_normal((t, h), dtype=np.float32))
    nw = bf16(1.0 + 0.1 * rng.standard_normal(h, dtype=np.float32))
    gu = ops.nvfp4_quantize_weight(ctx, to_dev(d["gate_up"]), True)
    dn = ops.nvfp4_quantize_weight(ctx, to_dev(d["down"]), False)
    shared = ops.SharedExpert(ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_gate_up"]), True),
                              ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_down"]), False), to_dev(d["sh_gate"]), s)
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, backend=ops.capi.MOE_BACKEND_NVFP4))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    outs = []
    for fused in (False, True):
        x, r = to_dev(d["hidden"]), to_dev(resid)
        out = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
        if fused:
            packed, tiled = ops.fused_add_rmsnorm_nvfp4(ctx, x, r, to_dev(nw), 1e-6, 1.0)
            ops.moe_layer_execute(plan, x, to_dev(d["router"]), gu, dn, out, ws, shared=shared,
                                  hidden_packed=packed, hidden_scale_tiled=tiled)
        else:
            ops.fused_add_rmsnorm(ctx, x, r, to_dev(nw), 1e-6)
            ops.moe_layer_execute(plan, x, to_dev(d["router"]), gu, dn, out, ws, shared=shared)
        torch.cuda.synchronize()
        assert ctx.read_device_error() == 0
        outs.append(to_np(out))
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("kind", ["nvfp4_shared", "bf16", "fp8"])
def test_layer_with_fused_post_norm(ops, ctx, oracle, kind):
    """Post-MoE residual add + next-layer RMSNorm folded into the combine == the layer call
    followed by qsfi_fused_add_rmsnorm: residual bit-exact, norm within one bf16 step (the
    row sum of squares is reduced in a different order)."""
    from helpers import make_moe_inputs
    t, h, e, k, i = 150, 512, 16, 4, 256
    s = 256 if kind == "nvfp4_shared" else 0
    d = make_moe_inputs(91, t, h, e, i, s)
    rng = d["rng"]
    resid = bf16(rng.standard_normal((t, h), dtype=np.float32))
    nw = bf16(1.0 + 0.1 * rng.standard_normal(h, dtype=np.float32))
    shared = None
    if kind == "nvfp4_shared":
        backend = ops.capi.MOE_BACKEND_NVFP4
        gu = ops.nvfp4_quantize_weight(ctx, to_dev(d["gate_up"]), True)
        dn = ops.nvfp4_quantize_weight(ctx, to_dev(d["down"]), False)
        shared = ops.SharedExpert(ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_gate_up"]), True),
                                  ops.nvfp4_quantize_weight(ctx, to_dev(d["sh_down"]), False),
                                  to_dev(d["sh_gate"]), s)
    elif kind == "fp8":
        backend = ops.capi.MOE_BACKEND_FP8_BLOCKSCALE
        gu, dn = ops.fp8_quantize_weight(ctx, to_dev(d["gate_up"])), ops.fp8_quantize_weight(ctx, to_dev(d["down"]))
    else:
        backend = ops.capi.MOE_BACKEND_STAGED_BF16
        gu, dn = to_dev(d["gate_up"]), to_dev(d["down"])
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=e, top_k=k, backend=backend))
    ws = torch.zeros(plan.layer_workspace_size(t, s), dtype=torch.uint8, device="cuda")
    x = to_dev(d["hidden"])
    # unfused: layer, then the stand-alone fused add + norm
    out_a = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    res_a = to_dev(resid)
    ops.moe_layer_execute(plan, x, to_dev(d["router"]), gu, dn, out_a, ws, shared=shared)
    moe_out = to_np(out_a)
    ops.fused_add_rmsnorm(ctx, out_a, res_a, to_dev(nw), 1e-6)
    # fused
    out_b = torch.empty((t, h), dtype=torch.bfloat16, device="cuda")
    res_b = to_dev(resid)
    ops.moe_layer_execute(plan, x, to_dev(d["router"]), gu, dn, out_b, ws, shared=shared,
                          residual_inout=res_b, next_norm_weight=to_dev(nw), next_norm_eps=1e-6)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    assert np.array_equal(to_np(res_b), to_np(res_a))
    want_norm, want_res = oracle.fused_add_rmsnorm(moe_out, resid, nw, 1e-6)
    assert np.max(np.abs(f32(to_np(res_b)) - want_res)) <= 0.04
    assert np.max(np.abs(f32(to_np(out_b)) - want_norm)) <= 0.06
    assert np.max(np.abs(f32(to_np(out_b)) - f32(to_np(out_a)))) <= 0.04   # at most one bf16 step apart
