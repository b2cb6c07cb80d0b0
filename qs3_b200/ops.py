"""Host-side operator layer over the C ABI, working on torch device tensors.

Mirrors the operator descriptors of the upstream runtime
(``src/runtime/kernels.rs:371-508,692-875``: ``RouterTopK``, ``MoeBf16PlanConfig``,
``MoeBf16Execute``, ``Bf16Gemm``, ``SiluAndMulBf16``,
``Qwen36SharedExpertGateAddBf16``) with the same argument meaning and the same
error classes: a failing call raises :class:`Qs3Error` carrying the
``qsfi_status`` and the context's last-error message, like the upstream
``Status`` results. torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import capi

_STATUS_NAMES = {0: "Ok", 1: "InvalidArgument", 2: "Unsupported", 3: "OutOfMemory",
                 4: "CudaError", 5: "BackendError", 6: "InternalError"}


class Qs3Error(RuntimeError):
    def __init__(self, status: int, message: str = ""):
        self.status = status
        self.message = message
        super().__init__(f"{_STATUS_NAMES.get(status, status)}: {message}")


_TORCH_DTYPES = {
    torch.float32: capi.DTYPE_F32, torch.float16: capi.DTYPE_F16, torch.bfloat16: capi.DTYPE_BF16,
    torch.int32: capi.DTYPE_I32, torch.int8: capi.DTYPE_I8, torch.uint8: capi.DTYPE_U8,
    torch.float8_e4m3fn: capi.DTYPE_FP8_E4M3,
}


def _desc(t, rank, dtype=None):
    """qsfi_tensorN view of a torch tensor (None -> absent optional tensor)."""
    cls = {1: capi.Tensor1, 2: capi.Tensor2, 3: capi.Tensor3}[rank]
    d = cls()
    if t is None:
        return d
    if t.dim() != rank:
        raise Qs3Error(capi.STATUS_INVALID_ARGUMENT, f"expected a rank-{rank} tensor, got {t.dim()}")
    d.data = t.data_ptr()
    d.dtype = dtype if dtype is not None else _TORCH_DTYPES.get(t.dtype, capi.DTYPE_INVALID)
    for i in range(rank):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def _stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class Context:
    """``qsfi_context``: device ordinal + stream + last-error record."""

    def __init__(self, device: int | None = None, stream: int | None = None, lib=None):
        self._lib = capi.load() if lib is None else lib   # lib: e.g. capi.load_checked()
        if device is None:
            device = torch.cuda.current_device()
        self.device = device
        if device < 0:   # no device binding: host-side calls only (validation, checkpoint parsing)
            desc = capi.ContextDesc(-1, None)
        else:
            desc = capi.ContextDesc(device, stream if stream is not None else _stream_ptr(device))
        handle = C.c_void_p()
        status = self._lib.qsfi_context_create(C.byref(desc), C.byref(handle))
        if status != capi.STATUS_OK:
            raise Qs3Error(status, "qsfi_context_create failed")
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self._lib.qsfi_context_destroy(self.handle)
            self.handle = None

    __del__ = close

    def set_stream(self, stream_ptr: int):
        self.check(self._lib.qsfi_context_set_stream(self.handle, C.c_void_p(stream_ptr)))

    def use_current_stream(self):
        self.set_stream(_stream_ptr(self.device))

    def last_error(self) -> capi.ErrorInfo:
        info = capi.ErrorInfo()
        self._lib.qsfi_context_get_last_error(self.handle, C.byref(info))
        return info

    def check(self, status: int):
        if status != capi.STATUS_OK:
            raise Qs3Error(status, self.last_error().message.decode(errors="replace"))

    def validate_target(self):
        self.check(self._lib.qsfi_context_validate_target(self.handle))

    def read_device_error(self) -> int:
        code = C.c_uint32(0)
        self.check(self._lib.qs3_moe_read_device_error(self.handle, C.byref(code)))
        return code.value

    def check_device_error(self):
        """Synchronise the stream; raise ``Qs3Error`` (BACKEND_ERROR) if a bounded device-side wait
        of an earlier call ran out (a lost load, tensor-core commit or peer rank)."""
        self.check(self._lib.qs3_moe_check_device_error(self.handle))


@dataclass
class MoePlanConfig:
    """Fields of ``qsfi_moe_plan_desc`` (upstream qsfi.h:222-236)."""
    max_num_tokens: int
    hidden_size: int
    intermediate_size: int
    num_experts: int
    top_k: int
    local_expert_offset: int = 0
    local_num_experts: int | None = None
    backend: int = capi.MOE_BACKEND_STAGED_BF16
    route_mode: int = capi.MOE_ROUTE_PRECOMPUTED_TOPK
    activation_dtype: int | None = None
    weight_dtype: int | None = None
    output_dtype: int = capi.DTYPE_BF16

    def to_c(self) -> capi.MoePlanDesc:
        nv = self.backend == capi.MOE_BACKEND_NVFP4
        f8 = self.backend == capi.MOE_BACKEND_FP8_BLOCKSCALE
        d = capi.MoePlanDesc()
        d.backend = self.backend
        d.route_mode = self.route_mode
        d.max_num_tokens = self.max_num_tokens
        d.hidden_size = self.hidden_size
        d.intermediate_size = self.intermediate_size
        d.num_experts = self.num_experts
        d.top_k = self.top_k
        d.local_expert_offset = self.local_expert_offset
        d.local_num_experts = self.num_experts if self.local_num_experts is None else self.local_num_experts
        default = capi.DTYPE_NVFP4_E2M1 if nv else capi.DTYPE_FP8_E4M3 if f8 else capi.DTYPE_BF16
        d.activation_dtype = default if self.activation_dtype is None else self.activation_dtype
        d.weight_dtype = default if self.weight_dtype is None else self.weight_dtype
        d.output_dtype = self.output_dtype
        return d


class MoePlan:
    def __init__(self, ctx: Context, config: MoePlanConfig):
        self.ctx = ctx
        self.config = config
        handle = C.c_void_p()
        desc = config.to_c()
        ctx.check(ctx._lib.qsfi_moe_plan_create(ctx.handle, C.byref(desc), C.byref(handle)))
        self.handle = handle
        self.desc = desc

    def close(self):
        if getattr(self, "handle", None):
            self.ctx._lib.qsfi_moe_plan_destroy(self.handle)
            self.handle = None

    __del__ = close

    def workspace_size(self, num_tokens: int) -> int:
        n = C.c_size_t(0)
        self.ctx.check(self.ctx._lib.qsfi_moe_workspace_size(self.ctx.handle, self.handle, num_tokens,
                                                             C.byref(n)))
        return n.value

    def layer_workspace_size(self, num_tokens: int, shared_intermediate_size: int = 0) -> int:
        n = C.c_size_t(0)
        self.ctx.check(self.ctx._lib.qs3_moe_layer_workspace_size(
            self.ctx.handle, self.handle, num_tokens, shared_intermediate_size, C.byref(n)))
        return n.value

    def routing_tables(self, workspace: torch.Tensor, num_tokens: int):
        """counts, indptr, route_rows, row_tokens, row_scales of the last execute."""
        view = capi.RoutingView()
        self.ctx.check(self.ctx._lib.qs3_moe_routing_tables(
            self.ctx.handle, self.handle, num_tokens, C.c_void_p(workspace.data_ptr()), C.byref(view)))
        e = self.desc.local_num_experts
        r = num_tokens * self.desc.top_k
        base = workspace.data_ptr()

        def grab(ptr, count, dtype):
            off = ptr - base
            return workspace[off:off + count * 4].view(dtype).clone()

        torch.cuda.synchronize()
        counts = grab(view.counts, e, torch.int32)
        indptr = grab(view.indptr, e + 1, torch.int32)
        route_rows = grab(view.route_rows, r, torch.int32)
        n = int(indptr[-1].item())
        row_tokens = grab(view.row_tokens, r, torch.int32)[:n]
        row_scales = grab(view.row_scales, r, torch.float32)[:n]
        return counts, indptr, route_rows, row_tokens, row_scales


# ------------------------------------------------------------------ qscu ops ---

def router_topk(logits, topk_ids, topk_weights, *, score=capi.ROUTER_SCORE_SOFTMAX, renormalize=True,
                routed_scaling_factor=1.0, num_tokens=None, num_experts=None, top_k=None, stream=None,
                lib=None):
    """``qscu_router_topk`` (upstream qscu.h:278; builder src/runtime/kernels.rs:692-741)."""
    lib = capi.load() if lib is None else lib
    d = capi.RouterTopkDesc()
    d.logits = _desc(logits, 2)
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.num_tokens = logits.shape[0] if num_tokens is None else num_tokens
    d.num_experts = logits.shape[1] if num_experts is None else num_experts
    d.top_k = topk_ids.shape[1] if top_k is None else top_k
    d.score = score
    d.renormalize = 1 if renormalize else 0
    d.routed_scaling_factor = routed_scaling_factor
    status = lib.qscu_router_topk(C.byref(d), C.c_void_p(_stream_ptr() if stream is None else stream))
    if status != capi.STATUS_OK:
        raise Qs3Error(status, "qscu_router_topk")


def silu_and_mul_bf16(gate, up, out, stream=None):
    """``qscu_silu_and_mul_bf16`` (upstream qscu.h:35)."""
    lib = capi.load()
    d = capi.SiluAndMulDesc()
    d.gate = _desc(gate, 2)
    d.up = _desc(up, 2)
    d.out = _desc(out, 2)
    d.num_tokens = out.shape[0]
    d.intermediate_size = out.shape[1]
    status = lib.qscu_silu_and_mul_bf16(C.byref(d), C.c_void_p(_stream_ptr() if stream is None else stream))
    if status != capi.STATUS_OK:
        raise Qs3Error(status, "qscu_silu_and_mul_bf16")


def shared_expert_gate_add_bf16(gate_logits, shared, out, stream=None):
    """``qscu_qwen36_shared_expert_gate_add_bf16`` (upstream qscu.h:50-52)."""
    lib = capi.load()
    d = capi.SharedExpertGateAddDesc()
    d.gate_logits = _desc(gate_logits, 2)
    d.shared = _desc(shared, 2)
    d.out = _desc(out, 2)
    d.num_tokens = out.shape[0]
    d.hidden_size = out.shape[1]
    status = lib.qscu_qwen36_shared_expert_gate_add_bf16(
        C.byref(d), C.c_void_p(_stream_ptr() if stream is None else stream))
    if status != capi.STATUS_OK:
        raise Qs3Error(status, "qscu_qwen36_shared_expert_gate_add_bf16")


# ------------------------------------------------------------------ qscb op ---

class GemmContext:
    """``qscb_context`` (upstream qscb.h:27-52)."""

    def __init__(self, device: int | None = None, stream: int | None = None):
        self._lib = capi.load()
        if device is None:
            device = torch.cuda.current_device()
        desc = capi.QscbContextDesc(device, stream if stream is not None else _stream_ptr(device))
        handle = C.c_void_p()
        status = self._lib.qscb_context_create(C.byref(desc), C.byref(handle))
        if status != capi.STATUS_OK:
            raise Qs3Error(status, "qscb_context_create failed")
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self._lib.qscb_context_destroy(self.handle)
            self.handle = None

    __del__ = close

    def gemm_bf16(self, x, weight, out, alpha=0.0, beta=0.0):
        """out = alpha * x @ weight.T + beta * out (``qscb_gemm_bf16``)."""
        d = capi.QscbGemmDesc()
        d.x = _desc(x, 2)
        d.weight = _desc(weight, 2)
        d.out = _desc(out, 2)
        d.rows = x.shape[0]
        d.in_features = x.shape[1]
        d.out_features = weight.shape[0]
        d.alpha = alpha
        d.beta = beta
        status = self._lib.qscb_gemm_bf16(self.handle, C.byref(d))
        if status != capi.STATUS_OK:
            info = capi.ErrorInfo()
            self._lib.qscb_context_get_last_error(self.handle, C.byref(info))
            raise Qs3Error(status, info.message.decode(errors="replace"))


# ------------------------------------------------------------------- MoE ops ---

def moe_execute_bf16(plan: MoePlan, hidden, topk_ids, topk_weights, gate_up_weight, down_weight, out,
                     workspace, num_tokens=None):
    """``qsfi_moe_execute_bf16`` (upstream qsfi.h:339-341)."""
    ctx = plan.ctx
    d = capi.MoeBf16ExecuteDesc()
    d.hidden = _desc(hidden, 2)
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.gate_up_weight = _desc(gate_up_weight, 3)
    d.down_weight = _desc(down_weight, 3)
    d.out = _desc(out, 2)
    d.workspace = _desc(workspace, 1)
    d.num_tokens = hidden.shape[0] if num_tokens is None else num_tokens
    ctx.check(ctx._lib.qsfi_moe_execute_bf16(ctx.handle, plan.handle, C.byref(d)))


def moe_execute_nvfp4(plan: MoePlan, hidden_packed, hidden_scale, topk_ids, topk_weights,
                      gate_up_weight_packed, gate_up_weight_scale, down_weight_packed, down_weight_scale,
                      out, workspace, expert_output_scale=None, num_tokens=None):
    """``qsfi_moe_execute_nvfp4`` (upstream qsfi.h:342-344; declared layout qsfi.h:249-266)."""
    ctx = plan.ctx
    d = capi.MoeNvfp4ExecuteDesc()
    d.hidden_packed = _desc(hidden_packed, 2)
    d.hidden_scale = _desc(hidden_scale, 2, capi.DTYPE_FP8_E4M3)
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.gate_up_weight_packed = _desc(gate_up_weight_packed, 3)
    d.gate_up_weight_scale = _desc(gate_up_weight_scale, 3, capi.DTYPE_FP8_E4M3)
    d.down_weight_packed = _desc(down_weight_packed, 3)
    d.down_weight_scale = _desc(down_weight_scale, 3, capi.DTYPE_FP8_E4M3)
    d.expert_output_scale = _desc(expert_output_scale, 1)
    d.out = _desc(out, 2)
    d.workspace = _desc(workspace, 1)
    d.num_tokens = hidden_packed.shape[0] if num_tokens is None else num_tokens
    ctx.check(ctx._lib.qsfi_moe_execute_nvfp4(ctx.handle, plan.handle, C.byref(d)))


@dataclass
class Nvfp4Weight:
    """Prepared NVFP4 weight: packed codes, linear and tiled scales, per-expert global scale."""
    packed: torch.Tensor        # u8 [E, rows, k/2]
    scale_linear: torch.Tensor  # u8 (e4m3 codes) [E, rows, k/16]
    scale_tiled: torch.Tensor   # u8 [E * tiled_bytes]
    global_scale: torch.Tensor  # f32 [E]


def nvfp4_tiled_scale_bytes(rows: int, k: int) -> int:
    return int(capi.load().qs3_nvfp4_tiled_scale_bytes(rows, k))


def nvfp4_quantize_weight(ctx: Context, weight: torch.Tensor, gated: bool, linear: bool = True) -> Nvfp4Weight:
    """``qs3_nvfp4_quantize_weight``: bf16 [E, rows, k] -> NVFP4."""
    e, rows, k = weight.shape
    dev = weight.device
    packed = torch.empty((e, rows, k // 2), dtype=torch.uint8, device=dev)
    sl = torch.empty((e, rows, k // 16), dtype=torch.uint8, device=dev) if linear else None
    st = torch.zeros(e * nvfp4_tiled_scale_bytes(rows, k), dtype=torch.uint8, device=dev)
    g = torch.empty(e, dtype=torch.float32, device=dev)
    d = capi.Nvfp4QuantizeWeightDesc()
    d.weight = _desc(weight, 3)
    d.packed = _desc(packed, 3)
    d.scale_linear = _desc(sl, 3, capi.DTYPE_FP8_E4M3)
    d.scale_tiled = _desc(st, 1)
    d.global_scale = _desc(g, 1)
    d.gated_rows = 1 if gated else 0
    ctx.check(ctx._lib.qs3_nvfp4_quantize_weight(ctx.handle, C.byref(d)))
    return Nvfp4Weight(packed, sl, st, g)


def nvfp4_quantize_act(ctx: Context, x: torch.Tensor, global_scale: float = 1.0):
    """``qs3_nvfp4_quantize_act``: bf16 [rows, k] -> (packed u8 [rows, k/2], e4m3 codes [rows, k/16])."""
    rows, k = x.shape
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty((rows, k // 16), dtype=torch.uint8, device=x.device)
    d = capi.Nvfp4QuantizeActDesc()
    d.x = _desc(x, 2)
    d.packed = _desc(packed, 2)
    d.scale_linear = _desc(scale, 2, capi.DTYPE_FP8_E4M3)
    d.global_scale = global_scale
    d.rows = rows
    ctx.check(ctx._lib.qs3_nvfp4_quantize_act(ctx.handle, C.byref(d)))
    return packed, scale


def nvfp4_tile_scales(ctx: Context, scale_linear: torch.Tensor, gated: bool) -> torch.Tensor:
    """``qs3_nvfp4_tile_scales``: e4m3 codes [E, rows, k/16] -> tiled buffer."""
    e, rows, kb = scale_linear.shape
    st = torch.zeros(e * nvfp4_tiled_scale_bytes(rows, kb * 16), dtype=torch.uint8, device=scale_linear.device)
    d = capi.Nvfp4TileScalesDesc()
    d.scale_linear = _desc(scale_linear, 3, capi.DTYPE_FP8_E4M3)
    d.scale_tiled = _desc(st, 1)
    d.gated_rows = 1 if gated else 0
    ctx.check(ctx._lib.qs3_nvfp4_tile_scales(ctx.handle, C.byref(d)))
    return st


@dataclass
class Fp8Weight:
    """Prepared FP8 weight: e4m3 codes and one f32 scale per 128 x 128 block."""
    codes: torch.Tensor  # u8 (e4m3 codes) [E, rows, k]
    scale: torch.Tensor  # f32 [E, ceil(rows/128), k/128]


def fp8_quantize_weight(ctx: Context, weight: torch.Tensor) -> Fp8Weight:
    """``qs3_fp8_quantize_weight``: bf16 [E, rows, k] -> e4m3 codes + 128 x 128 block scales."""
    e, rows, k = weight.shape
    codes = torch.empty((e, rows, k), dtype=torch.uint8, device=weight.device)
    scale = torch.empty((e, (rows + 127) // 128, k // 128), dtype=torch.float32, device=weight.device)
    d = capi.Fp8QuantizeWeightDesc()
    d.weight = _desc(weight, 3)
    d.codes = _desc(codes, 3, capi.DTYPE_FP8_E4M3)
    d.scale = _desc(scale, 3)
    ctx.check(ctx._lib.qs3_fp8_quantize_weight(ctx.handle, C.byref(d)))
    return Fp8Weight(codes, scale)


def fp8_quantize_act(ctx: Context, x: torch.Tensor):
    """``qs3_fp8_quantize_act``: bf16 [rows, k] -> (e4m3 codes u8 [rows, k], f32 [rows, k/128])."""
    rows, k = x.shape
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scale = torch.empty((rows, k // 128), dtype=torch.float32, device=x.device)
    d = capi.Fp8QuantizeActDesc()
    d.x = _desc(x, 2)
    d.codes = _desc(codes, 2, capi.DTYPE_FP8_E4M3)
    d.scale = _desc(scale, 2)
    d.rows = rows
    ctx.check(ctx._lib.qs3_fp8_quantize_act(ctx.handle, C.byref(d)))
    return codes, scale


def moe_execute_fp8(plan: MoePlan, hidden_codes, hidden_scale, topk_ids, topk_weights, gate_up: Fp8Weight,
                    down: Fp8Weight, out, workspace, num_tokens=None):
    """``qs3_moe_execute_fp8``: routed experts on FP8 block-scaled operands."""
    ctx = plan.ctx
    d = capi.MoeFp8ExecuteDesc()
    d.hidden = _desc(hidden_codes, 2, capi.DTYPE_FP8_E4M3)
    d.hidden_scale = _desc(hidden_scale, 2)
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.gate_up_weight = _desc(gate_up.codes, 3, capi.DTYPE_FP8_E4M3)
    d.gate_up_weight_scale = _desc(gate_up.scale, 3)
    d.down_weight = _desc(down.codes, 3, capi.DTYPE_FP8_E4M3)
    d.down_weight_scale = _desc(down.scale, 3)
    d.out = _desc(out, 2)
    d.workspace = _desc(workspace, 1)
    d.num_tokens = hidden_codes.shape[0] if num_tokens is None else num_tokens
    ctx.check(ctx._lib.qs3_moe_execute_fp8(ctx.handle, plan.handle, C.byref(d)))


@dataclass
class SharedExpert:
    """Shared-expert weights of one layer (upstream src/model.rs:963-968)."""
    gate_up: object          # bf16 [1, 2*Is, H] tensor or Nvfp4Weight
    down: object             # bf16 [1, H, Is] tensor or Nvfp4Weight
    gate_weight: torch.Tensor  # bf16 [1, H]
    intermediate_size: int


def moe_layer_execute(plan: MoePlan, hidden, router_weight, gate_up, down, out, workspace, *,
                      router_bias=None, shared: SharedExpert | None = None,
                      score=capi.ROUTER_SCORE_SOFTMAX, renormalize=True, routed_scaling_factor=1.0,
                      act_global_scale=1.0, act2_global_scale=1.0, topk_ids=None, topk_weights=None,
                      router_logits=None, num_tokens=None, hidden_packed=None, hidden_scale_tiled=None,
                      residual_inout=None, next_norm_weight=None, next_norm_eps=1e-6):
    """``qs3_moe_layer_execute``: the whole layer of upstream ``execute_moe_mlp``
    (src/model.rs:2072-2228) in one call. ``gate_up`` / ``down`` are bf16 tensors for
    a bf16 plan, :class:`Nvfp4Weight` for an NVFP4 plan and :class:`Fp8Weight` for an FP8
    block-scaled plan."""
    ctx = plan.ctx
    d = capi.MoeLayerDesc()
    d.hidden = _desc(hidden, 2)
    d.router_weight = _desc(router_weight, 2)
    d.router_bias = _desc(router_bias, 1)

    def put(prefix, w):
        if isinstance(w, Nvfp4Weight):
            setattr(d, f"{prefix}_weight", _desc(w.packed, 3))
            setattr(d, f"{prefix}_scale_tiled", _desc(w.scale_tiled, 1))
            setattr(d, f"{prefix}_global_scale", _desc(w.global_scale, 1))
        elif isinstance(w, Fp8Weight):
            setattr(d, f"{prefix}_weight", _desc(w.codes, 3, capi.DTYPE_FP8_E4M3))
            setattr(d, f"{prefix}_scale_tiled", _desc(w.scale.reshape(-1), 1))
        else:
            setattr(d, f"{prefix}_weight", _desc(w, 3))

    put("gate_up", gate_up)
    put("down", down)
    if shared is not None:
        put("shared_gate_up", shared.gate_up)
        put("shared_down", shared.down)
        d.shared_gate_weight = _desc(shared.gate_weight, 2)
        d.shared_intermediate_size = shared.intermediate_size
    d.score = score
    d.renormalize = 1 if renormalize else 0
    d.routed_scaling_factor = routed_scaling_factor
    d.act_global_scale = act_global_scale
    d.act2_global_scale = act2_global_scale
    d.out = _desc(out, 2)
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.router_logits = _desc(router_logits, 2)
    d.workspace = _desc(workspace, 1)
    d.num_tokens = hidden.shape[0] if num_tokens is None else num_tokens
    d.hidden_packed = _desc(hidden_packed, 2)
    d.hidden_scale_tiled = _desc(hidden_scale_tiled, 1)
    d.residual_inout = _desc(residual_inout, 2)
    d.next_norm_weight = _desc(next_norm_weight, 1)
    d.next_norm_eps = next_norm_eps
    ctx.check(ctx._lib.qs3_moe_layer_execute(ctx.handle, plan.handle, C.byref(d)))


def route_sort_static(ctx: Context, topk_ids, topk_weights, local_expert_offset: int,
                      local_num_experts: int, out=None):
    """``qs3_moe_route_sort_static``: the route permutation with library-resident scratch.

    For callers that may not allocate device memory when they need the routing tables
    (every byte of HBM already handed to fixed pools, or a section that cannot afford
    ``cudaMalloc``'s device-wide synchronisation). The five output tensors are the
    caller's and can be passed in as ``out=(counts, indptr, route_rows, row_tokens,
    row_scales)`` so that this wrapper allocates nothing either; without ``out`` it
    creates them with torch for convenience. At most 131072 routes and 1024 local
    experts; calls on one device must not overlap on the GPU (they share the scratch).
    Returns ``(counts, indptr, route_rows, row_tokens, row_scales)``; the last two are
    valid up to ``indptr[-1]`` entries.
    """
    t, k = topk_ids.shape
    dev = topk_ids.device
    if out is None:
        out = (torch.empty(local_num_experts, dtype=torch.int32, device=dev),
               torch.empty(local_num_experts + 1, dtype=torch.int32, device=dev),
               torch.empty(t * k, dtype=torch.int32, device=dev),
               torch.empty(t * k, dtype=torch.int32, device=dev),
               torch.empty(t * k, dtype=torch.float32, device=dev))
    d = capi.RouteSortStaticDesc()
    d.topk_ids = _desc(topk_ids, 2)
    d.topk_weights = _desc(topk_weights, 2)
    d.counts, d.indptr, d.route_rows, d.row_tokens, d.row_scales = (_desc(x, 1) for x in out)
    d.num_tokens, d.top_k = t, k
    d.local_expert_offset, d.local_num_experts = local_expert_offset, local_num_experts
    ctx.check(ctx._lib.qs3_moe_route_sort_static(ctx.handle, C.byref(d)))
    return out


# ------------------------------------------------------------ measurement aids ---

STAGE_NAMES = {1: "router_logits_gemm", 2: "router_topk", 3: "route_sort", 4: "gather_quantize",
               5: "gate_up_gemm_swiglu", 6: "down_gemm", 7: "shared_expert", 8: "combine"}


def ep_barrier(ctx: Context, pads, my_rank: int, epoch: int, timeout_cycles: int = 0, epoch_counter=None):
    """``qs3_moe_ep_barrier``: barrier over the ranks whose signal pads (device addresses as mapped
    here, one per rank) are ``pads``; bounded wait, see ``Context.check_device_error``. With
    ``epoch_counter`` (an int32 / uint32 device tensor of one element, zeroed once) the kernel counts
    the epochs itself, which makes the launch replayable from a CUDA graph."""
    d = capi.MoeEpBarrierDesc()
    arr = (C.c_void_p * len(pads))(*[int(p) for p in pads])
    d.pads, d.num_ranks, d.my_rank, d.epoch, d.timeout_cycles = arr, len(pads), my_rank, epoch & 0xFFFFFFFF, timeout_cycles
    if epoch_counter is not None:
        d.epoch_counter = epoch_counter.data_ptr()
    ctx.check(ctx._lib.qs3_moe_ep_barrier(ctx.handle, C.byref(d)))


def bounded_wait_probe(ctx: Context, limit_cycles: int = 100000):
    """``qs3_debug_bounded_wait_probe``: a kernel whose wait nothing satisfies; returns after the limit."""
    ctx.check(ctx._lib.qs3_debug_bounded_wait_probe(ctx.handle, limit_cycles))


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(capi.load().qs3_moe_launch_count())


def profile_begin(ctx: Context):
    ctx.check(ctx._lib.qs3_moe_profile_begin(ctx.handle))


def profile_end(ctx: Context):
    """[(stage name, ms), ...] for every stage recorded since ``profile_begin``."""
    cap = 64
    ids = (C.c_int32 * cap)()
    ms = (C.c_float * cap)()
    n = C.c_uint32(0)
    ctx.check(ctx._lib.qs3_moe_profile_end(ctx.handle, ids, ms, cap, C.byref(n)))
    return [(STAGE_NAMES.get(ids[i], str(ids[i])), float(ms[i])) for i in range(n.value)]


PEAK_KINDS = {"bf16": 0, "fp8": 1, "nvfp4": 2}


def tensor_peak_probe(ctx: Context, kind: str = "nvfp4", n: int = 256, iters: int = 20000,
                      pair: bool = False, cps_main: int = 0, cps_side: int = 0) -> float:
    """Dense TFLOP/s of back-to-back ``tcgen05.mma`` (128 x n tiles, operands resident in
    shared memory) on every SM: the tensor-pipe ceiling for one operand format. ``pair``:
    CTA pairs issuing ``cta_group::2`` instructions of 256 x n instead. ``cps_main`` /
    ``cps_side``: scale-tile copies per iteration of four MMAs issued by the MMA thread / by a
    second thread (NVFP4, single CTA)."""
    out = C.c_double(0.0)
    code = PEAK_KINDS[kind] + (16 if pair else 0) + 256 * cps_main + 4096 * cps_side
    ctx.check(ctx._lib.qs3_tensor_peak_probe(ctx.handle, code, n, iters, C.byref(out)))
    return float(out.value)


def operand_stream_probe(ctx: Context, buffer, tile_bytes: int = 16384, stages: int = 4, tiles: int = 2000,
                         boxes: bool = False) -> float:
    """``qs3_operand_stream_probe``: GB/s at which all SMs together stream ``buffer`` (a device tensor;
    L2-resident when it is smaller than the L2) into shared memory with bulk copies, ``stages`` tiles of
    ``tile_bytes`` in flight per SM: the operand-delivery ceiling of the streaming GEMMs. ``boxes``: every
    tile is a 128-row x 128-byte swizzled box of a matrix with 1 KiB rows instead of contiguous bytes."""
    out = C.c_double(0.0)
    ctx.check(ctx._lib.qs3_operand_stream_probe(ctx.handle, buffer.data_ptr(), buffer.numel() * buffer.element_size(),
                                                tile_bytes, stages, tiles, 1 if boxes else 0, C.byref(out)))
    return float(out.value)


def rmsnorm(ctx: Context, x, weight, out, eps: float = 1e-6, weight_bias: float = 0.0):
    """``qsfi_rmsnorm`` (upstream qsfi.h:160-167, 330)."""
    d = capi.RmsnormDesc()
    d.x, d.weight, d.out = _desc(x, 2), _desc(weight, 1), _desc(out, 2)
    d.hidden_size, d.weight_bias, d.eps = x.shape[1], weight_bias, eps
    ctx.check(ctx._lib.qsfi_rmsnorm(ctx.handle, C.byref(d)))


def _fused_desc(x, residual, weight, eps):
    d = capi.FusedAddRmsnormDesc()
    d.x, d.residual_inout, d.weight, d.out = _desc(x, 2), _desc(residual, 2), _desc(weight, 1), _desc(x, 2)
    d.hidden_size, d.eps = x.shape[1], eps
    return d


def fused_add_rmsnorm(ctx: Context, x, residual, weight, eps: float = 1e-6):
    """``qsfi_fused_add_rmsnorm`` (upstream qsfi.h:169-176, 331): residual += x; x = norm(residual)."""
    d = _fused_desc(x, residual, weight, eps)
    ctx.check(ctx._lib.qsfi_fused_add_rmsnorm(ctx.handle, C.byref(d)))


def fused_add_rmsnorm_nvfp4(ctx: Context, x, residual, weight, eps: float = 1e-6, global_scale: float = 1.0,
                            packed=None, tiled=None):
    """``qs3_fused_add_rmsnorm_nvfp4``: as above, and returns the NVFP4 codes and tiled scales
    of the normalised rows (token order). ``packed`` / ``tiled``: buffers to write into (a caller
    that replays a CUDA graph owns them); allocated here when absent."""
    rows, hidden = x.shape
    if packed is None:
        packed = torch.empty((rows, hidden // 2), dtype=torch.uint8, device=x.device)
    if tiled is None:
        tiled = torch.zeros(nvfp4_tiled_scale_bytes(rows, hidden), dtype=torch.uint8, device=x.device)
    d = capi.FusedAddRmsnormNvfp4Desc()
    d.norm = _fused_desc(x, residual, weight, eps)
    d.packed, d.scale_tiled, d.global_scale = _desc(packed, 2), _desc(tiled, 1), global_scale
    ctx.check(ctx._lib.qs3_fused_add_rmsnorm_nvfp4(ctx.handle, C.byref(d)))
    return packed, tiled
