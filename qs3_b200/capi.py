"""ctypes mirror of ``include/qs3_moe.h``.

The structures below have the same field order and types as the C declarations
(which in turn are layout-compatible with upstream ``qs_info.h``, ``qs_tensor.h``,
``qsfi.h``, ``qscu.h`` and ``qscb.h``). Loading fails loudly when the CUDA library
has not been built: there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libqs3moe.so")
CHECKED_LIB_PATH = os.path.join(PKG_DIR, "libqs3moe_checked.so")

ERROR_MESSAGE_BYTES = 512

# qsfi_status (upstream qs_info.h:20-28)
STATUS_OK = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_UNSUPPORTED = 2
STATUS_OUT_OF_MEMORY = 3
STATUS_CUDA_ERROR = 4
STATUS_BACKEND_ERROR = 5
STATUS_INTERNAL_ERROR = 6

# qsfi_dtype (upstream qs_tensor.h:15-29)
DTYPE_INVALID = 0
DTYPE_F32 = 1
DTYPE_F16 = 2
DTYPE_BF16 = 3
DTYPE_FP8_E4M3 = 4
DTYPE_FP8_E5M2 = 5
DTYPE_NVFP4_E2M1 = 6
DTYPE_MXFP4_E2M1 = 7
DTYPE_MXFP8_E4M3 = 8
DTYPE_I32 = 9
DTYPE_U32 = 10
DTYPE_I8 = 11
DTYPE_U8 = 12

MOE_BACKEND_STAGED_BF16 = 1
MOE_BACKEND_FUSED_BF16 = 2
MOE_BACKEND_NVFP4 = 3
MOE_BACKEND_FP8_BLOCKSCALE = 100  # QS3_MOE_BACKEND_FP8_BLOCKSCALE
MOE_ROUTE_PRECOMPUTED_TOPK = 0
MOE_ROUTE_ROUTER_LOGITS = 1
ROUTER_SCORE_SOFTMAX = 0
ROUTER_SCORE_SIGMOID = 1


class ErrorInfo(C.Structure):
    _fields_ = [("status", C.c_int), ("source", C.c_int), ("native_code", C.c_int32),
                ("message", C.c_char * ERROR_MESSAGE_BYTES)]


def _tensor(rank):
    class T(C.Structure):
        _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("shape", C.c_int64 * rank),
                    ("stride", C.c_int64 * rank)]
    T.__name__ = f"Tensor{rank}"
    return T


Tensor1 = _tensor(1)
Tensor2 = _tensor(2)
Tensor3 = _tensor(3)


class ContextDesc(C.Structure):
    _fields_ = [("device_ordinal", C.c_int32), ("stream", C.c_void_p)]


class BuildConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("target_sm", "target_compute_capability_major",
                                          "target_compute_capability_minor", "assume_fp8",
                                          "assume_fp4", "assume_pdl", "gemm_backend")]


class ContextInfo(C.Structure):
    _fields_ = [("runtime_compute_capability_major", C.c_uint32),
                ("runtime_compute_capability_minor", C.c_uint32)]


class MoePlanDesc(C.Structure):
    _fields_ = [("backend", C.c_int), ("route_mode", C.c_int), ("max_num_tokens", C.c_uint32),
                ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32),
                ("num_experts", C.c_uint32), ("top_k", C.c_uint32),
                ("local_expert_offset", C.c_uint32), ("local_num_experts", C.c_uint32),
                ("activation_dtype", C.c_int), ("weight_dtype", C.c_int), ("output_dtype", C.c_int),
                ("reserved0", C.c_uint32)]


class MoeBf16ExecuteDesc(C.Structure):
    _fields_ = [("hidden", Tensor2), ("topk_ids", Tensor2), ("topk_weights", Tensor2),
                ("gate_up_weight", Tensor3), ("down_weight", Tensor3), ("out", Tensor2),
                ("workspace", Tensor1), ("num_tokens", C.c_uint32)]


class MoeNvfp4ExecuteDesc(C.Structure):
    _fields_ = [("hidden_packed", Tensor2), ("hidden_scale", Tensor2), ("topk_ids", Tensor2),
                ("topk_weights", Tensor2), ("gate_up_weight_packed", Tensor3),
                ("gate_up_weight_scale", Tensor3), ("down_weight_packed", Tensor3),
                ("down_weight_scale", Tensor3), ("expert_output_scale", Tensor1), ("out", Tensor2),
                ("workspace", Tensor1), ("num_tokens", C.c_uint32)]


class RouterTopkDesc(C.Structure):
    _fields_ = [("logits", Tensor2), ("topk_ids", Tensor2), ("topk_weights", Tensor2),
                ("num_tokens", C.c_uint32), ("num_experts", C.c_uint32), ("top_k", C.c_uint32),
                ("score", C.c_int), ("renormalize", C.c_uint32), ("routed_scaling_factor", C.c_float)]


class SiluAndMulDesc(C.Structure):
    _fields_ = [("gate", Tensor2), ("up", Tensor2), ("out", Tensor2), ("num_tokens", C.c_uint32),
                ("intermediate_size", C.c_uint32)]


class SharedExpertGateAddDesc(C.Structure):
    _fields_ = [("gate_logits", Tensor2), ("shared", Tensor2), ("out", Tensor2),
                ("num_tokens", C.c_uint32), ("hidden_size", C.c_uint32)]


class QscbContextDesc(C.Structure):
    _fields_ = [("device_ordinal", C.c_int32), ("stream", C.c_void_p)]


class QscbGemmDesc(C.Structure):
    _fields_ = [("x", Tensor2), ("weight", Tensor2), ("out", Tensor2), ("rows", C.c_uint32),
                ("in_features", C.c_uint32), ("out_features", C.c_uint32), ("alpha", C.c_float),
                ("beta", C.c_float), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class Nvfp4QuantizeWeightDesc(C.Structure):
    _fields_ = [("weight", Tensor3), ("packed", Tensor3), ("scale_linear", Tensor3),
                ("scale_tiled", Tensor1), ("global_scale", Tensor1), ("gated_rows", C.c_uint32)]


class Nvfp4QuantizeActDesc(C.Structure):
    _fields_ = [("x", Tensor2), ("packed", Tensor2), ("scale_linear", Tensor2),
                ("global_scale", C.c_float), ("rows", C.c_uint32)]


class Nvfp4TileScalesDesc(C.Structure):
    _fields_ = [("scale_linear", Tensor3), ("scale_tiled", Tensor1), ("gated_rows", C.c_uint32)]


class MoeLayerDesc(C.Structure):
    _fields_ = [("hidden", Tensor2), ("router_weight", Tensor2), ("router_bias", Tensor1),
                ("gate_up_weight", Tensor3), ("gate_up_scale_tiled", Tensor1),
                ("gate_up_global_scale", Tensor1), ("down_weight", Tensor3),
                ("down_scale_tiled", Tensor1), ("down_global_scale", Tensor1),
                ("shared_gate_up_weight", Tensor3), ("shared_gate_up_scale_tiled", Tensor1),
                ("shared_gate_up_global_scale", Tensor1), ("shared_down_weight", Tensor3),
                ("shared_down_scale_tiled", Tensor1), ("shared_down_global_scale", Tensor1),
                ("shared_gate_weight", Tensor2), ("shared_intermediate_size", C.c_uint32),
                ("score", C.c_int), ("renormalize", C.c_uint32), ("routed_scaling_factor", C.c_float),
                ("act_global_scale", C.c_float), ("act2_global_scale", C.c_float), ("out", Tensor2),
                ("topk_ids", Tensor2), ("topk_weights", Tensor2), ("router_logits", Tensor2),
                ("workspace", Tensor1), ("num_tokens", C.c_uint32), ("hidden_packed", Tensor2),
                ("hidden_scale_tiled", Tensor1), ("residual_inout", Tensor2), ("next_norm_weight", Tensor1),
                ("next_norm_eps", C.c_float)]


class MoeEpRouteDesc(C.Structure):
    _fields_ = [("hidden", Tensor2), ("router_weight", Tensor2), ("router_bias", Tensor1),
                ("router_logits", Tensor2), ("topk_ids", Tensor2), ("topk_weights", Tensor2),
                ("hidden_packed", Tensor2), ("hidden_scale", Tensor2), ("score", C.c_int),
                ("renormalize", C.c_uint32), ("routed_scaling_factor", C.c_float),
                ("act_global_scale", C.c_float), ("num_tokens", C.c_uint32),
                ("expert_id_map", Tensor1), ("dispatch_ids", Tensor2), ("rank_mask", Tensor1),
                ("num_ranks", C.c_uint32)]


class MoeNvfp4PreparedDesc(C.Structure):
    _fields_ = [("hidden_packed", Tensor2), ("hidden_scale", Tensor2), ("topk_ids", Tensor2),
                ("topk_weights", Tensor2), ("gate_up_weight", Tensor3), ("gate_up_scale_tiled", Tensor1),
                ("gate_up_global_scale", Tensor1), ("down_weight", Tensor3), ("down_scale_tiled", Tensor1),
                ("down_global_scale", Tensor1), ("act_global_scale", C.c_float),
                ("act2_global_scale", C.c_float), ("out", Tensor2), ("workspace", Tensor1),
                ("num_tokens", C.c_uint32), ("flags", C.c_uint32)]


class MoeEpFinishDesc(C.Structure):
    _fields_ = [("hidden", Tensor2), ("partials", Tensor3), ("shared_gate_up_weight", Tensor3),
                ("shared_gate_up_scale_tiled", Tensor1), ("shared_gate_up_global_scale", Tensor1),
                ("shared_down_weight", Tensor3), ("shared_down_scale_tiled", Tensor1),
                ("shared_down_global_scale", Tensor1), ("shared_gate_weight", Tensor2),
                ("shared_intermediate_size", C.c_uint32), ("act_global_scale", C.c_float),
                ("act2_global_scale", C.c_float), ("out", Tensor2), ("workspace", Tensor1),
                ("num_tokens", C.c_uint32), ("num_ranks", C.c_uint32), ("phases", C.c_uint32),
                ("peer_partials", C.POINTER(C.c_void_p)), ("topk_ids", Tensor2)]


class RoutingView(C.Structure):
    _fields_ = [("counts", C.c_void_p), ("indptr", C.c_void_p), ("route_rows", C.c_void_p),
                ("row_tokens", C.c_void_p), ("row_scales", C.c_void_p)]


ROUTE_SORT_STATIC_MAX_ROUTES = 131072
ROUTE_SORT_STATIC_MAX_EXPERTS = 1024


class RouteSortStaticDesc(C.Structure):
    _fields_ = [("topk_ids", Tensor2), ("topk_weights", Tensor2), ("counts", Tensor1),
                ("indptr", Tensor1), ("route_rows", Tensor1), ("row_tokens", Tensor1),
                ("row_scales", Tensor1), ("num_tokens", C.c_uint32), ("top_k", C.c_uint32),
                ("local_expert_offset", C.c_uint32), ("local_num_experts", C.c_uint32)]


# Every symbol include/qs3_moe.h declares: (restype, argtypes)
_P = C.POINTER
class Fp8QuantizeWeightDesc(C.Structure):
    _fields_ = [("weight", Tensor3), ("codes", Tensor3), ("scale", Tensor3)]


class Fp8QuantizeActDesc(C.Structure):
    _fields_ = [("x", Tensor2), ("codes", Tensor2), ("scale", Tensor2), ("rows", C.c_uint32)]


class MoeFp8ExecuteDesc(C.Structure):
    _fields_ = [("hidden", Tensor2), ("hidden_scale", Tensor2), ("topk_ids", Tensor2),
                ("topk_weights", Tensor2), ("gate_up_weight", Tensor3), ("gate_up_weight_scale", Tensor3),
                ("down_weight", Tensor3), ("down_weight_scale", Tensor3), ("out", Tensor2),
                ("workspace", Tensor1), ("num_tokens", C.c_uint32)]


class MoeEpPullTokensDesc(C.Structure):
    _fields_ = [("peer_blocks", _P(C.c_void_p)), ("segment_offset", C.c_uint64 * 4),
                ("segment_bytes", C.c_uint64 * 4), ("dst", C.c_void_p * 4), ("num_ranks", C.c_uint32),
                ("num_segments", C.c_uint32)]


class MoeEpPullRoutedDesc(C.Structure):
    _fields_ = [("peer_blocks", _P(C.c_void_p)), ("offset_codes", C.c_uint64), ("offset_scales", C.c_uint64),
                ("offset_ids", C.c_uint64), ("offset_weights", C.c_uint64), ("offset_mask", C.c_uint64),
                ("dst_codes", C.c_void_p), ("dst_scales", C.c_void_p), ("dst_ids", C.c_void_p),
                ("dst_weights", C.c_void_p), ("num_ranks", C.c_uint32), ("my_rank", C.c_uint32),
                ("num_tokens", C.c_uint32), ("top_k", C.c_uint32), ("hidden_size", C.c_uint32)]


class MoeEpBarrierDesc(C.Structure):
    _fields_ = [("pads", _P(C.c_void_p)), ("num_ranks", C.c_uint32), ("my_rank", C.c_uint32),
                ("epoch", C.c_uint32), ("timeout_cycles", C.c_uint64), ("epoch_counter", C.c_void_p)]


class RmsnormDesc(C.Structure):
    _fields_ = [("x", Tensor2), ("weight", Tensor1), ("out", Tensor2), ("hidden_size", C.c_uint32),
                ("weight_bias", C.c_float), ("eps", C.c_float)]


class FusedAddRmsnormDesc(C.Structure):
    _fields_ = [("x", Tensor2), ("residual_inout", Tensor2), ("weight", Tensor1), ("out", Tensor2),
                ("hidden_size", C.c_uint32), ("eps", C.c_float)]


class FusedAddRmsnormNvfp4Desc(C.Structure):
    _fields_ = [("norm", FusedAddRmsnormDesc), ("packed", Tensor2), ("scale_tiled", Tensor1),
                ("global_scale", C.c_float)]


CHECKPOINT_MAX_RANK = 8
CHECKPOINT_EXPERTS_BF16_FUSED = 0
CHECKPOINT_EXPERTS_NVFP4_SPLIT = 1


class CheckpointTensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("file", C.c_char_p), ("dtype_name", C.c_char_p), ("dtype", C.c_int),
                ("element_bytes", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_int64 * CHECKPOINT_MAX_RANK),
                ("file_offset", C.c_uint64), ("bytes", C.c_uint64)]


class CheckpointMoeConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32), ("num_experts", C.c_uint32),
                ("top_k", C.c_uint32), ("shared_intermediate_size", C.c_uint32), ("num_layers", C.c_uint32),
                ("renormalize", C.c_uint32), ("rms_norm_eps", C.c_float)]


class MoeLayerLoadDesc(C.Structure):
    _fields_ = [("layer_prefix", C.c_char_p), ("hidden_size", C.c_uint32), ("intermediate_size", C.c_uint32),
                ("num_experts", C.c_uint32), ("shared_intermediate_size", C.c_uint32),
                ("local_expert_offset", C.c_uint32), ("local_num_experts", C.c_uint32),
                ("expert_order", _P(C.c_uint32)), ("format", C.c_int), ("backend", C.c_int),
                ("fused_transposed", C.c_uint32)]


class MoeLayerWeights(C.Structure):
    _fields_ = [("router_weight", Tensor2),
                ("gate_up_weight", Tensor3), ("gate_up_scale_tiled", Tensor1), ("gate_up_global_scale", Tensor1),
                ("down_weight", Tensor3), ("down_scale_tiled", Tensor1), ("down_global_scale", Tensor1),
                ("shared_gate_up_weight", Tensor3), ("shared_gate_up_scale_tiled", Tensor1),
                ("shared_gate_up_global_scale", Tensor1),
                ("shared_down_weight", Tensor3), ("shared_down_scale_tiled", Tensor1),
                ("shared_down_global_scale", Tensor1),
                ("shared_gate_weight", Tensor2),
                ("act_global_scale", C.c_float), ("act2_global_scale", C.c_float)]


_SIGNATURES = {
    "qsfi_status_string": (C.c_char_p, [C.c_int]),
    "qsfi_context_create": (C.c_int, [_P(ContextDesc), _P(C.c_void_p)]),
    "qsfi_context_destroy": (None, [C.c_void_p]),
    "qsfi_context_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "qsfi_get_build_config": (C.c_int, [_P(BuildConfig)]),
    "qsfi_context_get_info": (C.c_int, [C.c_void_p, _P(ContextInfo)]),
    "qsfi_context_validate_target": (C.c_int, [C.c_void_p]),
    "qsfi_context_get_last_error": (C.c_int, [C.c_void_p, _P(ErrorInfo)]),
    "qsfi_context_clear_last_error": (None, [C.c_void_p]),
    "qsfi_moe_plan_create": (C.c_int, [C.c_void_p, _P(MoePlanDesc), _P(C.c_void_p)]),
    "qsfi_moe_plan_destroy": (None, [C.c_void_p]),
    "qsfi_moe_workspace_size": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, _P(C.c_size_t)]),
    "qsfi_moe_execute_bf16": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeBf16ExecuteDesc)]),
    "qsfi_moe_execute_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeNvfp4ExecuteDesc)]),
    "qscu_router_topk": (C.c_int, [_P(RouterTopkDesc), C.c_void_p]),
    "qscu_silu_and_mul_bf16": (C.c_int, [_P(SiluAndMulDesc), C.c_void_p]),
    "qscu_qwen36_shared_expert_gate_add_bf16": (C.c_int, [_P(SharedExpertGateAddDesc), C.c_void_p]),
    "qscb_context_create": (C.c_int, [_P(QscbContextDesc), _P(C.c_void_p)]),
    "qscb_context_destroy": (None, [C.c_void_p]),
    "qscb_context_get_last_error": (C.c_int, [C.c_void_p, _P(ErrorInfo)]),
    "qscb_context_clear_last_error": (None, [C.c_void_p]),
    "qscb_gemm_bf16": (C.c_int, [C.c_void_p, _P(QscbGemmDesc)]),
    "qs3_nvfp4_tiled_scale_bytes": (C.c_size_t, [C.c_uint64, C.c_uint64]),
    "qs3_nvfp4_quantize_weight": (C.c_int, [C.c_void_p, _P(Nvfp4QuantizeWeightDesc)]),
    "qs3_nvfp4_quantize_act": (C.c_int, [C.c_void_p, _P(Nvfp4QuantizeActDesc)]),
    "qs3_nvfp4_tile_scales": (C.c_int, [C.c_void_p, _P(Nvfp4TileScalesDesc)]),
    "qs3_moe_layer_workspace_size": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                               _P(C.c_size_t)]),
    "qs3_moe_layer_execute": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeLayerDesc)]),
    "qs3_moe_routing_tables": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
                                         _P(RoutingView)]),
    "qs3_moe_route_sort_static": (C.c_int, [C.c_void_p, _P(RouteSortStaticDesc)]),
    "qs3_moe_ep_route": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeEpRouteDesc)]),
    "qs3_moe_execute_nvfp4_prepared": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeNvfp4PreparedDesc)]),
    "qs3_moe_ep_finish_workspace_size": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
                                                   _P(C.c_size_t)]),
    "qs3_moe_ep_finish": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeEpFinishDesc)]),
    "qs3_moe_ep_pull_tokens": (C.c_int, [C.c_void_p, _P(MoeEpPullTokensDesc)]),
    "qsfi_rmsnorm": (C.c_int, [C.c_void_p, _P(RmsnormDesc)]),
    "qsfi_fused_add_rmsnorm": (C.c_int, [C.c_void_p, _P(FusedAddRmsnormDesc)]),
    "qs3_fused_add_rmsnorm_nvfp4": (C.c_int, [C.c_void_p, _P(FusedAddRmsnormNvfp4Desc)]),
    "qs3_moe_ep_pull_routed": (C.c_int, [C.c_void_p, _P(MoeEpPullRoutedDesc)]),
    "qs3_moe_ep_barrier": (C.c_int, [C.c_void_p, _P(MoeEpBarrierDesc)]),
    "qs3_moe_read_device_error": (C.c_int, [C.c_void_p, _P(C.c_uint32)]),
    "qs3_moe_check_device_error": (C.c_int, [C.c_void_p]),
    "qs3_debug_bounded_wait_probe": (C.c_int, [C.c_void_p, C.c_uint64]),
    "qs3_debug_pair_trace": (C.c_int, [_P(C.c_uint64), C.c_uint32, _P(C.c_uint32)]),
    "qs3_debug_pair_spans": (C.c_int, [_P(C.c_uint64), C.c_uint32]),
    "qs3_moe_launch_count": (C.c_uint64, []),
    "qs3_moe_profile_begin": (C.c_int, [C.c_void_p]),
    "qs3_moe_profile_end": (C.c_int, [C.c_void_p, _P(C.c_int32), _P(C.c_float), C.c_uint32,
                                      _P(C.c_uint32)]),
    "qs3_fp8_quantize_weight": (C.c_int, [C.c_void_p, _P(Fp8QuantizeWeightDesc)]),
    "qs3_fp8_quantize_act": (C.c_int, [C.c_void_p, _P(Fp8QuantizeActDesc)]),
    "qs3_moe_execute_fp8": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeFp8ExecuteDesc)]),
    "qsfi_moe_execute_fp8": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeFp8ExecuteDesc)]),
    "qs3_tensor_peak_probe": (C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, _P(C.c_double)]),
    "qs3_operand_stream_probe": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32,
                                           C.c_uint32, _P(C.c_double)]),
    "qs3_checkpoint_open": (C.c_int, [C.c_void_p, C.c_char_p, _P(C.c_void_p)]),
    "qs3_checkpoint_close": (None, [C.c_void_p]),
    "qs3_checkpoint_num_tensors": (C.c_uint64, [C.c_void_p]),
    "qs3_checkpoint_tensor_at": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, _P(CheckpointTensorInfo)]),
    "qs3_checkpoint_find": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p, _P(CheckpointTensorInfo)]),
    "qs3_checkpoint_read_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]),
    "qs3_checkpoint_read_moe_config": (C.c_int, [C.c_void_p, C.c_void_p, _P(CheckpointMoeConfig)]),
    "qs3_checkpoint_moe_layer_bytes": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeLayerLoadDesc), _P(C.c_size_t),
                                                 _P(C.c_size_t)]),
    "qs3_checkpoint_load_moe_layer": (C.c_int, [C.c_void_p, C.c_void_p, _P(MoeLayerLoadDesc), C.c_void_p, C.c_size_t,
                                                C.c_void_p, C.c_size_t, _P(MoeLayerWeights)]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None
_checked_lib = None


def _bind(path: str) -> C.CDLL:
    lib = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


def load() -> C.CDLL:
    """Load ``libqs3moe.so``; raises when it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m qs3_b200._build` "
                "(nvcc, sm_100a). There is no CPU or library fallback for this path.")
        _lib = _bind(LIB_PATH)
    return _lib


def load_checked() -> C.CDLL:
    """Load ``libqs3moe_checked.so``, the build with device-side input validation
    (``QSFI_ENABLE_CHECKED_VALIDATION=1``: one stream sync per validated call)."""
    global _checked_lib
    if _checked_lib is None:
        if not os.path.exists(CHECKED_LIB_PATH):
            raise RuntimeError(f"{CHECKED_LIB_PATH} is missing: build it with `python -m qs3_b200._build`.")
        _checked_lib = _bind(CHECKED_LIB_PATH)
    return _checked_lib
