"""CPU-side checks of the C ABI: the library loads, exports every symbol the header
declares, struct layouts match the C side, and descriptor validation fails with
upstream's status classes and message fragments *before any device addressing*
(fake device pointers, as in tests_cuda_qscu_gdn_router.inc:112-115)."""
import ctypes as C
import os
import re

import pytest

from qs3_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _fake(tag):
    return 0x1000 + tag * 0x1000


def _t(cls, ptr, dtype, shape, stride=None):
    t = cls()
    t.data = ptr
    t.dtype = dtype
    n = len(shape)
    if stride is None:
        stride = [1] * n
        for i in range(n - 2, -1, -1):
            stride[i] = stride[i + 1] * shape[i + 1]
    for i in range(n):
        t.shape[i] = shape[i]
        t.stride[i] = stride[i]
    return t


@pytest.fixture(scope="module")
def lib():
    return capi.load()


@pytest.fixture()
def ctx(lib):
    handle = C.c_void_p()
    desc = capi.ContextDesc(-1, None)  # no device binding: pure host validation
    assert lib.qsfi_context_create(C.byref(desc), C.byref(handle)) == capi.STATUS_OK
    yield handle
    lib.qsfi_context_destroy(handle)


def _message(lib, ctx):
    info = capi.ErrorInfo()
    lib.qsfi_context_get_last_error(ctx, C.byref(info))
    return info.status, info.message.decode()


def _plan_desc(**kw):
    d = capi.MoePlanDesc()
    d.backend = capi.MOE_BACKEND_STAGED_BF16
    d.route_mode = capi.MOE_ROUTE_PRECOMPUTED_TOPK
    d.max_num_tokens, d.hidden_size, d.intermediate_size = 16, 256, 128
    d.num_experts, d.top_k, d.local_expert_offset, d.local_num_experts = 8, 2, 0, 8
    d.activation_dtype = d.weight_dtype = d.output_dtype = capi.DTYPE_BF16
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def test_header_symbols_are_exported(lib):
    header = open(os.path.join(ROOT, "include", "qs3_moe.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b((?:qsfi|qscu|qscb|qs3)_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(capi.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    checked = capi.load_checked()     # the checked-validation build exports the same interface
    for name in declared:
        assert hasattr(checked, name), name


def test_struct_sizes_match_the_c_side():
    # x86-64 SysV layout of the C declarations
    assert C.sizeof(capi.ErrorInfo) == 12 + 512
    assert C.sizeof(capi.Tensor1) == 32 and C.sizeof(capi.Tensor2) == 48 and C.sizeof(capi.Tensor3) == 64
    assert C.sizeof(capi.MoePlanDesc) == 52
    assert C.sizeof(capi.MoeBf16ExecuteDesc) == 48 * 4 + 64 * 2 + 32 + 8
    assert C.sizeof(capi.RouterTopkDesc) == 48 * 3 + 24


def test_status_strings_and_build_config(lib):
    assert lib.qsfi_status_string(0) == b"ok" and lib.qsfi_status_string(2) == b"unsupported"
    assert lib.qsfi_status_string(99) == b"unknown status"
    cfg = capi.BuildConfig()
    assert lib.qsfi_get_build_config(C.byref(cfg)) == capi.STATUS_OK
    assert (cfg.target_sm, cfg.target_compute_capability_major, cfg.target_compute_capability_minor) == (100, 10, 0)
    assert lib.qsfi_get_build_config(None) == capi.STATUS_INVALID_ARGUMENT


def test_plan_validation(lib, ctx):
    plan = C.c_void_p()
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc()), None) == capi.STATUS_INVALID_ARGUMENT
    assert lib.qsfi_moe_plan_create(None, C.byref(_plan_desc()), C.byref(plan)) == capi.STATUS_INVALID_ARGUMENT
    assert lib.qsfi_moe_plan_create(ctx, None, C.byref(plan)) == capi.STATUS_INVALID_ARGUMENT
    assert "desc is null" in _message(lib, ctx)[1]
    for kw, status, frag in (
        (dict(top_k=0), capi.STATUS_INVALID_ARGUMENT, "non-zero"),
        (dict(local_expert_offset=4, local_num_experts=8), capi.STATUS_INVALID_ARGUMENT, "local expert range"),
        (dict(hidden_size=12), capi.STATUS_INVALID_ARGUMENT, "divisible by 8"),
        (dict(weight_dtype=capi.DTYPE_F16), capi.STATUS_INVALID_ARGUMENT, "bf16 activation"),
        (dict(backend=capi.MOE_BACKEND_FUSED_BF16), capi.STATUS_UNSUPPORTED, "unsupported MoE backend"),
        (dict(backend=capi.MOE_BACKEND_NVFP4), capi.STATUS_INVALID_ARGUMENT, "nvfp4 activation/weight"),
        (dict(top_k=40, num_experts=64, local_num_experts=64), capi.STATUS_UNSUPPORTED, "top_k"),
        (dict(backend=capi.MOE_BACKEND_FP8_BLOCKSCALE), capi.STATUS_INVALID_ARGUMENT, "fp8_e4m3 activation/weight"),
        (dict(backend=capi.MOE_BACKEND_FP8_BLOCKSCALE, activation_dtype=capi.DTYPE_FP8_E4M3,
              weight_dtype=capi.DTYPE_FP8_E4M3, hidden_size=192), capi.STATUS_INVALID_ARGUMENT,
         "divisible by 128"),
        (dict(backend=capi.MOE_BACKEND_FP8_BLOCKSCALE, activation_dtype=capi.DTYPE_FP8_E4M3,
              weight_dtype=capi.DTYPE_FP8_E4M3, hidden_size=8192), capi.STATUS_UNSUPPORTED, "up to 4096"),
    ):
        assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc(**kw)), C.byref(plan)) == status, kw
        assert frag in _message(lib, ctx)[1], kw
        assert not plan.value
    # expert-parallel plans are accepted by this build (upstream rejects them)
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc(local_expert_offset=4, local_num_experts=4)),
                                    C.byref(plan)) == capi.STATUS_OK
    lib.qsfi_moe_plan_destroy(plan)
    lib.qsfi_moe_plan_destroy(None)  # legal, like upstream
    # FP8 block-scaled plans (no upstream counterpart): workspace scales with 16-row token tiles
    fp8 = _plan_desc(backend=capi.MOE_BACKEND_FP8_BLOCKSCALE, activation_dtype=capi.DTYPE_FP8_E4M3,
                     weight_dtype=capi.DTYPE_FP8_E4M3)
    assert lib.qsfi_moe_plan_create(ctx, C.byref(fp8), C.byref(plan)) == capi.STATUS_OK
    n = C.c_size_t(0)
    assert lib.qsfi_moe_workspace_size(ctx, plan, 16, C.byref(n)) == capi.STATUS_OK
    assert n.value % 256 == 0 and n.value > 16 * 2 * (256 + 128 + 2 * 256)
    lib.qsfi_moe_plan_destroy(plan)


def _upstream_workspace(tokens, hidden, inter, experts, top_k):
    """The formula of upstream compute_workspace_layout (qsfi_moe.cu:67-121)."""
    r = tokens * top_k
    off = 0
    for count, size in ((experts, 4), (experts + 1, 4), (experts, 4), (r, 4), (r, 4), (r, 4),
                        (r * hidden, 2), (r * 2 * inter, 2), (r * inter, 2), (r * hidden, 2),
                        (experts * 3, 4)) + ((experts, 8),) * 6:
        off = (off + 255) // 256 * 256 + count * size
    return (off + 255) // 256 * 256


def test_workspace_size(lib, ctx):
    plan = C.c_void_p()
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc()), C.byref(plan)) == capi.STATUS_OK
    n = C.c_size_t(0)
    assert lib.qsfi_moe_workspace_size(ctx, plan, 16, C.byref(n)) == capi.STATUS_OK
    assert _upstream_workspace(16, 256, 128, 8, 2) == 60672  # the figure upstream reports for this shape
    assert n.value >= 60672 and n.value % 256 == 0
    assert lib.qsfi_moe_workspace_size(ctx, plan, 17, C.byref(n)) == capi.STATUS_INVALID_ARGUMENT
    assert "max_num_tokens" in _message(lib, ctx)[1]
    assert lib.qsfi_moe_workspace_size(ctx, plan, 16, None) == capi.STATUS_INVALID_ARGUMENT
    assert lib.qsfi_moe_workspace_size(ctx, None, 16, C.byref(n)) == capi.STATUS_INVALID_ARGUMENT
    lib.qsfi_moe_plan_destroy(plan)


def _bf16_execute_desc(tokens=16, hidden=256, inter=128, experts=8, top_k=2, ws=1 << 24):
    d = capi.MoeBf16ExecuteDesc()
    d.hidden = _t(capi.Tensor2, _fake(1), capi.DTYPE_BF16, [tokens, hidden])
    d.topk_ids = _t(capi.Tensor2, _fake(2), capi.DTYPE_I32, [tokens, top_k])
    d.topk_weights = _t(capi.Tensor2, _fake(3), capi.DTYPE_F32, [tokens, top_k])
    d.gate_up_weight = _t(capi.Tensor3, _fake(4), capi.DTYPE_BF16, [experts, 2 * inter, hidden])
    d.down_weight = _t(capi.Tensor3, _fake(5), capi.DTYPE_BF16, [experts, hidden, inter])
    d.out = _t(capi.Tensor2, _fake(6), capi.DTYPE_BF16, [tokens, hidden])
    d.workspace = _t(capi.Tensor1, _fake(7), capi.DTYPE_U8, [ws])
    d.num_tokens = tokens
    return d


def test_execute_bf16_validation_precedes_device_access(lib, ctx):
    plan = C.c_void_p()
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc()), C.byref(plan)) == capi.STATUS_OK
    assert lib.qsfi_moe_execute_bf16(None, plan, C.byref(_bf16_execute_desc())) == capi.STATUS_INVALID_ARGUMENT
    assert lib.qsfi_moe_execute_bf16(ctx, None, C.byref(_bf16_execute_desc())) == capi.STATUS_INVALID_ARGUMENT
    assert "plan/desc is null" in _message(lib, ctx)[1]

    def expect(mutate, frag, status=capi.STATUS_INVALID_ARGUMENT):
        d = _bf16_execute_desc()
        mutate(d)
        assert lib.qsfi_moe_execute_bf16(ctx, plan, C.byref(d)) == status, frag
        assert frag in _message(lib, ctx)[1], (frag, _message(lib, ctx))

    expect(lambda d: setattr(d, "num_tokens", 0), "invalid MoE num_tokens")
    expect(lambda d: setattr(d, "num_tokens", 17), "invalid MoE num_tokens")
    expect(lambda d: setattr(d.hidden, "data", None), "hidden.data must not be null")
    expect(lambda d: setattr(d.topk_ids, "dtype", capi.DTYPE_U32), "topk_ids dtype")
    expect(lambda d: d.out.shape.__setitem__(1, 0), "out shape/stride entries must be positive")
    expect(lambda d: setattr(d.workspace, "dtype", capi.DTYPE_F32), "workspace dtype must be u8 or i8")
    expect(lambda d: d.hidden.stride.__setitem__(0, 512), "hidden must be contiguous")
    expect(lambda d: d.down_weight.stride.__setitem__(2, 2), "down_weight must be contiguous")
    expect(lambda d: d.topk_ids.shape.__setitem__(1, 3) or d.topk_ids.stride.__setitem__(0, 3),
           "token/top-k tensor shape mismatch")
    expect(lambda d: d.gate_up_weight.shape.__setitem__(0, 4), "expert weight shape mismatch")
    expect(lambda d: d.workspace.shape.__setitem__(0, 1024), "workspace is too small")
    lib.qsfi_moe_plan_destroy(plan)

    nv = C.c_void_p()
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc(
        backend=capi.MOE_BACKEND_NVFP4, activation_dtype=capi.DTYPE_NVFP4_E2M1,
        weight_dtype=capi.DTYPE_NVFP4_E2M1)), C.byref(nv)) == capi.STATUS_OK
    assert lib.qsfi_moe_execute_bf16(ctx, nv, C.byref(_bf16_execute_desc())) == capi.STATUS_INVALID_ARGUMENT
    assert "requires a staged BF16 MoE plan" in _message(lib, ctx)[1]
    lib.qsfi_moe_plan_destroy(nv)


def test_execute_nvfp4_validation(lib, ctx):
    bf = C.c_void_p()
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc()), C.byref(bf)) == capi.STATUS_OK
    d = capi.MoeNvfp4ExecuteDesc()
    assert lib.qsfi_moe_execute_nvfp4(ctx, bf, C.byref(d)) == capi.STATUS_INVALID_ARGUMENT
    assert "requires an NVFP4 MoE plan" in _message(lib, ctx)[1]  # upstream test.cu:1736-1773 fragment
    assert lib.qsfi_moe_execute_nvfp4(ctx, None, C.byref(d)) == capi.STATUS_INVALID_ARGUMENT
    lib.qsfi_moe_plan_destroy(bf)
    nv = C.c_void_p()
    # hidden 256 / inter 128: a valid NVFP4 plan, but not a shape the tensor-core path tiles
    assert lib.qsfi_moe_plan_create(ctx, C.byref(_plan_desc(
        backend=capi.MOE_BACKEND_NVFP4, activation_dtype=capi.DTYPE_NVFP4_E2M1,
        weight_dtype=capi.DTYPE_NVFP4_E2M1)), C.byref(nv)) == capi.STATUS_OK
    d.num_tokens = 16
    assert lib.qsfi_moe_execute_nvfp4(ctx, nv, C.byref(d)) == capi.STATUS_INVALID_ARGUMENT
    assert "hidden_packed.data must not be null" in _message(lib, ctx)[1]
    lib.qsfi_moe_plan_destroy(nv)


def _router_desc(tokens=4, experts=16, top_k=2, logits_dtype=capi.DTYPE_F32):
    d = capi.RouterTopkDesc()
    d.logits = _t(capi.Tensor2, _fake(1), logits_dtype, [tokens, experts])
    d.topk_ids = _t(capi.Tensor2, _fake(2), capi.DTYPE_I32, [tokens, top_k])
    d.topk_weights = _t(capi.Tensor2, _fake(3), capi.DTYPE_F32, [tokens, top_k])
    d.num_tokens, d.num_experts, d.top_k = tokens, experts, top_k
    d.score, d.renormalize, d.routed_scaling_factor = 0, 1, 1.0
    return d


def test_router_validation_status_codes(lib):
    # upstream validate_router_desc, qscu.cu:1190-1224
    assert lib.qscu_router_topk(None, None) == capi.STATUS_INVALID_ARGUMENT
    for mutate, status in (
        (lambda d: setattr(d, "top_k", 0), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: setattr(d, "top_k", 17), capi.STATUS_UNSUPPORTED),
        (lambda d: setattr(d, "num_experts", 4097), capi.STATUS_UNSUPPORTED),
        (lambda d: setattr(d, "top_k", 16) or setattr(d, "num_experts", 8), capi.STATUS_UNSUPPORTED),
        (lambda d: setattr(d, "score", 2), capi.STATUS_UNSUPPORTED),
        (lambda d: setattr(d, "routed_scaling_factor", 0.0), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: setattr(d, "routed_scaling_factor", float("inf")), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: setattr(d.logits, "dtype", capi.DTYPE_F16), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: setattr(d.topk_ids, "data", None), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: d.logits.stride.__setitem__(0, 32), capi.STATUS_INVALID_ARGUMENT),
        (lambda d: d.topk_weights.shape.__setitem__(0, 3), capi.STATUS_INVALID_ARGUMENT),
    ):
        d = _router_desc()
        mutate(d)
        assert lib.qscu_router_topk(C.byref(d), None) == status


def test_elementwise_validation_status_codes(lib):
    d = capi.SiluAndMulDesc()
    assert lib.qscu_silu_and_mul_bf16(None, None) == capi.STATUS_INVALID_ARGUMENT
    assert lib.qscu_silu_and_mul_bf16(C.byref(d), None) == capi.STATUS_INVALID_ARGUMENT
    d.gate = _t(capi.Tensor2, _fake(1), capi.DTYPE_BF16, [2, 3])
    d.up = _t(capi.Tensor2, _fake(2), capi.DTYPE_BF16, [2, 3])
    d.out = _t(capi.Tensor2, _fake(3), capi.DTYPE_BF16, [2, 4])
    d.num_tokens, d.intermediate_size = 2, 3
    assert lib.qscu_silu_and_mul_bf16(C.byref(d), None) == capi.STATUS_INVALID_ARGUMENT
    g = capi.SharedExpertGateAddDesc()
    assert lib.qscu_qwen36_shared_expert_gate_add_bf16(C.byref(g), None) == capi.STATUS_INVALID_ARGUMENT
    g.gate_logits = _t(capi.Tensor2, _fake(1), capi.DTYPE_F16, [3, 1])
    g.shared = _t(capi.Tensor2, _fake(2), capi.DTYPE_BF16, [3, 4])
    g.out = _t(capi.Tensor2, _fake(3), capi.DTYPE_BF16, [3, 4])
    g.num_tokens, g.hidden_size = 3, 4
    assert lib.qscu_qwen36_shared_expert_gate_add_bf16(C.byref(g), None) == capi.STATUS_INVALID_ARGUMENT
    g.gate_logits = _t(capi.Tensor2, _fake(1), capi.DTYPE_F32, [3, 2])
    assert lib.qscu_qwen36_shared_expert_gate_add_bf16(C.byref(g), None) == capi.STATUS_INVALID_ARGUMENT


def test_tiled_scale_bytes_matches_oracle(lib, oracle):
    for rows, k in ((128, 256), (1024, 2048), (130, 512), (2048, 512)):
        assert lib.qs3_nvfp4_tiled_scale_bytes(rows, k) == oracle.tiled_scale_bytes(rows, k)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", "/nonexistent/libqs3moe.so")
    with pytest.raises(RuntimeError, match="no CPU or library fallback"):
        capi.load()


def test_header_compiles_as_c_and_cpp(tmp_path):
    """include/qs3_moe.h is the drop-in boundary: it must be plain C (the upstream bindgen input
    is C) and also valid C++, with no warnings under -Wall -Wextra -pedantic."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "hdr_check.c"
    src.write_text('#include "qs3_moe.h"\nint main(void) { qsfi_moe_plan_desc d; (void)d; '
                   "return (int)sizeof(qs3_moe_layer_desc) == 0; }\n")
    for compiler, flags in (("gcc", ["-std=c11", "-pedantic"]), ("g++", ["-std=c++17", "-x", "c++"])):
        exe = shutil.which(compiler)
        if exe is None:
            pytest.skip(f"{compiler} not installed")
        r = subprocess.run([exe, *flags, "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                            "-I", os.path.join(root, "include"), str(src)], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_reference_arm_layer_shapes_equal_the_workload_constants():
    """bench.py's reference arm imports neither torch nor the package, so it carries its own copy of
    the benchmark layer shapes; they must stay equal to qs3_b200.workload's."""
    import bench
    from qs3_b200 import workload
    ref = bench._RefConfigs.make()
    for name in ("PREFILL_NVFP4", "EP_NVFP4", "DECODE_NVFP4", "DECODE_FP8"):
        a, b = getattr(ref, name), getattr(workload, name)
        for field in ("name", "tokens", "hidden", "experts", "top_k", "inter", "shared_inter", "nvfp4", "zipf_s",
                      "fp8", "dtype_name"):
            assert getattr(a, field) == getattr(b, field), (name, field)
