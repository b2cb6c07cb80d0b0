"""ctypes/numpy binding of ``oracle/libqs3oracle.so`` (test infrastructure only).

Every function takes and returns numpy arrays; bf16 tensors travel as uint16 bit
patterns, e4m3 / packed e2m1 tensors as uint8.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqs3oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the recipe in ``oracle/Makefile``."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "qs3_oracle.cpp"))
    ):
        subprocess.run(["make", "-C", _HERE, "-B", "libqs3oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.qs3o_f32_to_bf16.restype = C.c_uint16
        _lib.qs3o_f32_to_bf16.argtypes = [C.c_float]
        _lib.qs3o_bf16_to_f32.restype = C.c_float
        _lib.qs3o_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.qs3o_f32_to_e4m3.restype = C.c_uint8
        _lib.qs3o_f32_to_e4m3.argtypes = [C.c_float]
        _lib.qs3o_e4m3_to_f32.restype = C.c_float
        _lib.qs3o_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.qs3o_f32_to_e2m1.restype = C.c_uint8
        _lib.qs3o_f32_to_e2m1.argtypes = [C.c_float]
        _lib.qs3o_e2m1_to_f32.restype = C.c_float
        _lib.qs3o_e2m1_to_f32.argtypes = [C.c_uint8]
        _lib.qs3o_num_threads.restype = C.c_int
        for name in ("qs3o_tiled_scale_bytes", "qs3o_tiled_scale_offset", "qs3o_gated_tiled_row"):
            getattr(_lib, name).restype = C.c_int64
        _lib.qs3o_tiled_scale_bytes.argtypes = [C.c_int64, C.c_int64]
        _lib.qs3o_tiled_scale_offset.argtypes = [C.c_int64, C.c_int64, C.c_int64]
        _lib.qs3o_gated_tiled_row.argtypes = [C.c_int64, C.c_int64]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().qs3o_num_threads())


def set_num_threads(n: int | None = None) -> int:
    """Use ``n`` OpenMP threads from now on (default: every core this process may run on)."""
    if n is None:
        n = len(os.sched_getaffinity(0))
    lib().qs3o_set_num_threads(C.c_int(int(n)))
    return num_threads()


# ----------------------------------------------------------------- codecs ---

def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even bf16 bit patterns (uint16) of a float32 array."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bits = bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    return (bits >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def e4m3_to_f32(c: np.ndarray) -> np.ndarray:
    table = np.array([lib().qs3o_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return table[np.asarray(c, dtype=np.uint8)]


def e2m1_to_f32(c: np.ndarray) -> np.ndarray:
    table = np.array([lib().qs3o_e2m1_to_f32(i) for i in range(16)], dtype=np.float32)
    return table[np.asarray(c, dtype=np.uint8) & 0xF]


# ----------------------------------------------------------------- router ---

def router_topk(logits, top_k, score=0, renormalize=True, scaling=1.0, bias=None):
    logits = _c(logits, np.float32)
    t, e = logits.shape
    ids = np.empty((t, top_k), np.int32)
    w = np.empty((t, top_k), np.float32)
    bias = _c(bias, np.float32)
    lib().qs3o_router_topk(_p(logits), C.c_int64(t), C.c_int64(e), C.c_int64(top_k), C.c_int(score),
                           C.c_int(1 if renormalize else 0), C.c_float(scaling), _p(bias), _p(ids), _p(w))
    return ids, w


def route_sort(ids, weights, local_offset, local_experts):
    ids = _c(ids, np.int32)
    weights = _c(weights, np.float32)
    t, k = ids.shape
    counts = np.zeros(local_experts, np.int32)
    indptr = np.zeros(local_experts + 1, np.int32)
    route_rows = np.empty(t * k, np.int32)
    row_tokens = np.full(t * k, -1, np.int32)
    row_scales = np.zeros(t * k, np.float32)
    lib().qs3o_route_sort(_p(ids), _p(weights), C.c_int64(t), C.c_int64(k), C.c_int64(local_offset),
                          C.c_int64(local_experts), _p(counts), _p(indptr), _p(route_rows),
                          _p(row_tokens), _p(row_scales))
    n = int(indptr[-1])
    return counts, indptr, route_rows, row_tokens[:n], row_scales[:n]


# ----------------------------------------------------------- element-wise ---

def silu_and_mul_bf16(gate, up):
    gate = _c(gate, np.uint16)
    up = _c(up, np.uint16)
    out = np.empty_like(gate)
    lib().qs3o_silu_and_mul_bf16(_p(gate), _p(up), C.c_int64(gate.size), _p(out))
    return out


def shared_gate_add_bf16(gate_logits, shared, out):
    gate_logits = _c(gate_logits, np.float32).reshape(-1)
    shared = _c(shared, np.uint16)
    out = np.array(out, dtype=np.uint16, copy=True)
    t, h = shared.shape
    lib().qs3o_shared_gate_add_bf16(_p(gate_logits), _p(shared), C.c_int64(t), C.c_int64(h), _p(out))
    return out


def gemm_bf16(x, w, out_dtype="f32", alpha=1.0, beta=0.0, out=None):
    x = _c(x, np.uint16)
    w = _c(w, np.uint16)
    rows, k = x.shape
    n = w.shape[0]
    if out_dtype == "f32":
        o = np.zeros((rows, n), np.float32) if out is None else np.array(out, np.float32, copy=True)
        lib().qs3o_gemm_bf16(_p(x), _p(w), C.c_int64(rows), C.c_int64(k), C.c_int64(n),
                             C.c_float(alpha), C.c_float(beta), _p(o), None)
    else:
        o = np.zeros((rows, n), np.uint16) if out is None else np.array(out, np.uint16, copy=True)
        lib().qs3o_gemm_bf16(_p(x), _p(w), C.c_int64(rows), C.c_int64(k), C.c_int64(n),
                             C.c_float(alpha), C.c_float(beta), None, _p(o))
    return o


# --------------------------------------------------------------- bf16 MoE ---

def moe_bf16(hidden, ids, weights, gate_up, down, local_offset=0, token_list=None):
    hidden = _c(hidden, np.uint16)
    ids = _c(ids, np.int32)
    weights = _c(weights, np.float32)
    gate_up = _c(gate_up, np.uint16)
    down = _c(down, np.uint16)
    t, h = hidden.shape
    e, two_i, _ = gate_up.shape
    k = ids.shape[1]
    tl = _c(token_list, np.int32)
    n = t if tl is None else tl.size
    out = np.empty((n, h), np.uint16)
    lib().qs3o_moe_bf16(_p(hidden), _p(ids), _p(weights), _p(gate_up), _p(down), C.c_int64(t),
                        C.c_int64(h), C.c_int64(two_i // 2), C.c_int64(k), C.c_int64(local_offset),
                        C.c_int64(e), _p(tl), C.c_int64(n), _p(out))
    return out


def shared_expert_bf16(hidden, gate_up, down, gate_w, out, token_list=None):
    hidden = _c(hidden, np.uint16)
    gate_up = _c(gate_up, np.uint16).reshape(-1, hidden.shape[1])
    down = _c(down, np.uint16).reshape(hidden.shape[1], -1)
    gate_w = _c(gate_w, np.uint16).reshape(-1)
    out = np.array(out, dtype=np.uint16, copy=True)
    t, h = hidden.shape
    tl = _c(token_list, np.int32)
    n = t if tl is None else tl.size
    lib().qs3o_shared_expert_bf16(_p(hidden), _p(gate_up), _p(down), _p(gate_w), C.c_int64(t),
                                  C.c_int64(h), C.c_int64(gate_up.shape[0] // 2), _p(tl),
                                  C.c_int64(n), _p(out))
    return out


# ------------------------------------------------------------------ NVFP4 ---

def tiled_scale_bytes(rows, k):
    return int(lib().qs3o_tiled_scale_bytes(rows, k))


def tiled_scale_index(rows, k, gated_inter=0):
    """int64 [rows, k/16] array: byte offset of every scale in the tiled layout."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    if gated_inter:
        up = r >= gated_inter
        i = np.where(up, r - gated_inter, r)
        r = (i // 64) * 128 + np.where(up, 64, 0) + i % 64
    kb = np.arange(k // 16, dtype=np.int64)[None, :]
    return ((r // 128) * (k // 64) + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4


def nvfp4_quantize_act(x, global_scale=1.0):
    x = _c(x, np.uint16)
    rows, k = x.shape
    packed = np.empty((rows, k // 2), np.uint8)
    scale = np.empty((rows, k // 16), np.uint8)
    lib().qs3o_nvfp4_quantize_act(_p(x), C.c_int64(rows), C.c_int64(k), C.c_float(global_scale),
                                  _p(packed), _p(scale))
    return packed, scale


def nvfp4_quantize_weight(w, gated=False, tiled=True):
    w = _c(w, np.uint16)
    e, rows, k = w.shape
    packed = np.empty((e, rows, k // 2), np.uint8)
    scale = np.empty((e, rows, k // 16), np.uint8)
    tb = tiled_scale_bytes(rows, k)
    st = np.zeros(e * tb, np.uint8) if tiled else None
    g = np.empty(e, np.float32)
    lib().qs3o_nvfp4_quantize_weight(_p(w), C.c_int64(e), C.c_int64(rows), C.c_int64(k),
                                     C.c_int(1 if gated else 0), _p(packed), _p(scale), _p(st), _p(g))
    return packed, scale, st, g


def nvfp4_dequantize(packed, scale, global_scale=None):
    """float32 values of packed e2m1 rows with linear e4m3 block scales."""
    packed = np.asarray(packed, np.uint8)
    lo = e2m1_to_f32(packed & 0xF)
    hi = e2m1_to_f32(packed >> 4)
    vals = np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    s = np.repeat(e4m3_to_f32(scale), 16, axis=-1)
    out = vals * s
    if global_scale is not None:
        g = np.asarray(global_scale, np.float32)
        out = out * g.reshape(g.shape + (1,) * (out.ndim - g.ndim))
    return out.astype(np.float32)


def moe_nvfp4(hidden_packed, hidden_scale, ids, weights, gu, d, *, act_global=1.0, act2_global=1.0,
              local_offset=0, shared=None, hidden_bf16=None, token_list=None):
    """``gu`` / ``d`` are (packed, scale_linear, global) triples; ``shared`` is
    None or a dict with keys gu, d (triples with one expert) and gate_w (bf16 [H])."""
    hp = _c(hidden_packed, np.uint8)
    hs = _c(hidden_scale, np.uint8)
    ids = _c(ids, np.int32)
    weights = _c(weights, np.float32)
    gup, gus, gug = (_c(gu[0], np.uint8), _c(gu[1], np.uint8), _c(gu[2], np.float32))
    dp, ds, dg = (_c(d[0], np.uint8), _c(d[1], np.uint8), _c(d[2], np.float32))
    t = hp.shape[0]
    h = hp.shape[1] * 2
    e, two_i, _ = gup.shape
    # globals of shape [2, experts] (routed) and [2] (shared): gate rows and up rows scaled apart
    split = int(gug.size == 2 * e)
    k = ids.shape[1]
    tl = _c(token_list, np.int32)
    n = t if tl is None else tl.size
    out = np.empty((n, h), np.uint16)
    if shared is not None:
        sgu = [_c(shared["gu"][0], np.uint8), _c(shared["gu"][1], np.uint8), _c(shared["gu"][2], np.float32)]
        sd = [_c(shared["d"][0], np.uint8), _c(shared["d"][1], np.uint8), _c(shared["d"][2], np.float32)]
        gate_w = _c(shared["gate_w"], np.uint16).reshape(-1)
        hb = _c(hidden_bf16, np.uint16)
        s_inter = sgu[0].reshape(-1, h // 2).shape[0] // 2
        split |= 2 * (sgu[2].size == 2)
    else:
        sgu = [None] * 3
        sd = [None] * 3
        gate_w = None
        hb = None
        s_inter = 0
    lib().qs3o_moe_nvfp4(_p(hp), _p(hs), C.c_float(act_global), C.c_float(act2_global), _p(ids),
                         _p(weights), _p(gup), _p(gus), _p(gug), _p(dp), _p(ds), _p(dg), C.c_int64(t),
                         C.c_int64(h), C.c_int64(two_i // 2), C.c_int64(k), C.c_int64(local_offset),
                         C.c_int64(e), _p(sgu[0]), _p(sgu[1]), _p(sgu[2]), _p(sd[0]), _p(sd[1]),
                         _p(sd[2]), C.c_int64(s_inter), _p(hb), _p(gate_w), _p(tl), C.c_int64(n),
                         C.c_int32(split), _p(out))
    return out


def fp8_quantize_act(x):
    """bf16 [rows, k] -> (e4m3 codes u8 [rows, k], f32 scales [rows, k/128])."""
    x = _c(x, np.uint16)
    rows, k = x.shape
    assert k % 128 == 0
    codes = np.empty((rows, k), np.uint8)
    scale = np.empty((rows, k // 128), np.float32)
    lib().qs3o_fp8_quantize_act(_p(x), C.c_int64(rows), C.c_int64(k), _p(codes), _p(scale))
    return codes, scale


def fp8_quantize_weight(w):
    """bf16 [experts, rows, k] -> (e4m3 codes, f32 scales [experts, ceil(rows/128), k/128])."""
    w = _c(w, np.uint16)
    e, rows, k = w.shape
    assert k % 128 == 0
    codes = np.empty((e, rows, k), np.uint8)
    scale = np.empty((e, (rows + 127) // 128, k // 128), np.float32)
    lib().qs3o_fp8_quantize_weight(_p(w), C.c_int64(e), C.c_int64(rows), C.c_int64(k), _p(codes), _p(scale))
    return codes, scale


def fp8_dequantize(codes, scale):
    """float32 values of e4m3 codes [..., rows, k] with [..., ceil(rows/128) or rows, k/128] scales."""
    codes = np.asarray(codes, np.uint8)
    vals = e4m3_to_f32(codes)
    s = np.repeat(np.asarray(scale, np.float32), 128, axis=-1)
    if s.shape[-2] != codes.shape[-2]:
        s = np.repeat(s, 128, axis=-2)[..., : codes.shape[-2], :]
    return (vals * s).astype(np.float32)


def moe_fp8(hidden_codes, hidden_scale, ids, weights, gu, d, *, local_offset=0, token_list=None):
    """``gu`` / ``d`` are (codes, scale) pairs of the expert weights."""
    hc = _c(hidden_codes, np.uint8)
    hs = _c(hidden_scale, np.float32)
    ids = _c(ids, np.int32)
    weights = _c(weights, np.float32)
    guc, gus = _c(gu[0], np.uint8), _c(gu[1], np.float32)
    dc, ds = _c(d[0], np.uint8), _c(d[1], np.float32)
    t, h = hc.shape
    e, two_i, _ = guc.shape
    k = ids.shape[1]
    tl = _c(token_list, np.int32)
    n = t if tl is None else tl.size
    out = np.empty((n, h), np.uint16)
    lib().qs3o_moe_fp8(_p(hc), _p(hs), _p(ids), _p(weights), _p(guc), _p(gus), _p(dc), _p(ds),
                       C.c_int64(t), C.c_int64(h), C.c_int64(two_i // 2), C.c_int64(k),
                       C.c_int64(local_offset), C.c_int64(e), _p(tl), C.c_int64(n), _p(out))
    return out


# ------------------------------------------------------------------ norms ---

def _norm_input(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return a, 1
    return a.astype(np.float32, copy=False), 0


def rmsnorm(x, weight, eps=1e-6, weight_bias=0.0):
    """f32 [rows, hidden] of the upstream RMSNorm checker; x / weight bf16 bits or f32."""
    x, is_bf16 = _norm_input(x)
    weight, _ = _norm_input(weight)
    rows, hidden = x.shape
    out = np.empty((rows, hidden), np.float32)
    lib().qs3o_rmsnorm(_p(x), _p(weight), C.c_int(is_bf16), C.c_int64(rows), C.c_int64(hidden),
                       C.c_float(eps), C.c_float(weight_bias), _p(out))
    return out


def fused_add_rmsnorm(x, residual, weight, eps=1e-6):
    """(norm f32, residual f32) of the upstream fused add + RMSNorm checker."""
    x, is_bf16 = _norm_input(x)
    residual, _ = _norm_input(residual)
    weight, _ = _norm_input(weight)
    rows, hidden = x.shape
    norm = np.empty((rows, hidden), np.float32)
    res = np.empty((rows, hidden), np.float32)
    lib().qs3o_fused_add_rmsnorm(_p(x), _p(residual), _p(weight), C.c_int(is_bf16), C.c_int64(rows),
                                 C.c_int64(hidden), C.c_float(eps), _p(norm), _p(res))
    return norm, res
