"""Checkpoint loader: safetensors shards -> the device tensors of one MoE layer.

Python face of the ``qs3_checkpoint_*`` entry points. Upstream has this component only
as a trait with four operations (``src/weight_loader.rs:33-38``) and a written contract
(``src/weight_loader.rs:9-32``, ``AGENTS.md:55-67``): every shard header, the index and
``config.json`` are parsed and checked before any device memory is touched; the bytes then
go from the files through a pinned staging ring into their final device storage.

Parsing, validation and sizing (`Checkpoint`, `Checkpoint.layer_bytes`) make no CUDA call
and work on a machine without a GPU; `load_moe_layer` needs one.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi
from .ops import Context, Nvfp4Weight, SharedExpert

_NUMPY_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64,
                 "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "U16": np.uint16,
                 "U32": np.uint32, "U64": np.uint64, "BOOL": np.uint8, "F8_E4M3": np.uint8, "F8_E5M2": np.uint8}


@dataclass(frozen=True)
class TensorInfo:
    """One entry of a shard header."""
    name: str
    file: str
    dtype: str            # safetensors spelling
    shape: tuple
    file_offset: int      # absolute offset inside the shard
    nbytes: int


def _info(raw: capi.CheckpointTensorInfo) -> TensorInfo:
    return TensorInfo(raw.name.decode(), raw.file.decode(), raw.dtype_name.decode(),
                      tuple(int(raw.shape[i]) for i in range(raw.rank)), int(raw.file_offset), int(raw.bytes))


class Checkpoint:
    """``qs3_checkpoint``: the parsed and validated headers of a checkpoint directory."""

    def __init__(self, ctx: Context, directory: str):
        self.ctx = ctx
        self._lib = ctx._lib
        handle = C.c_void_p()
        ctx.check(self._lib.qs3_checkpoint_open(ctx.handle, str(directory).encode(), C.byref(handle)))
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self._lib.qs3_checkpoint_close(self.handle)
            self.handle = None

    __del__ = close

    def __len__(self) -> int:
        return int(self._lib.qs3_checkpoint_num_tensors(self.handle))

    def tensors(self) -> list[TensorInfo]:
        out = []
        raw = capi.CheckpointTensorInfo()
        for i in range(len(self)):
            self.ctx.check(self._lib.qs3_checkpoint_tensor_at(self.ctx.handle, self.handle, i, C.byref(raw)))
            out.append(_info(raw))
        return out

    def find(self, name: str) -> TensorInfo:
        raw = capi.CheckpointTensorInfo()
        self.ctx.check(self._lib.qs3_checkpoint_find(self.ctx.handle, self.handle, name.encode(), C.byref(raw)))
        return _info(raw)

    def read_host(self, name: str) -> np.ndarray:
        """The tensor's bytes as a numpy array (bf16 and fp8 types as their bit patterns)."""
        info = self.find(name)
        out = np.empty(info.shape, dtype=_NUMPY_DTYPES[info.dtype])
        self.ctx.check(self._lib.qs3_checkpoint_read_host(self.ctx.handle, self.handle, name.encode(),
                                                          out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def moe_config(self) -> capi.CheckpointMoeConfig:
        cfg = capi.CheckpointMoeConfig()
        self.ctx.check(self._lib.qs3_checkpoint_read_moe_config(self.ctx.handle, self.handle, C.byref(cfg)))
        return cfg

    # ---- one MoE layer ----------------------------------------------------------------

    def _layer_desc(self, prefix, hidden, inter, experts, shared_inter, fmt, backend, local, expert_order,
                    fused_transposed):
        d = capi.MoeLayerLoadDesc()
        d.layer_prefix = prefix.encode()
        d.hidden_size, d.intermediate_size, d.num_experts = hidden, inter, experts
        d.shared_intermediate_size = shared_inter
        off, count = local if local is not None else (0, experts)
        d.local_expert_offset, d.local_num_experts = off, count
        keep = None
        if expert_order is not None:
            keep = (C.c_uint32 * len(expert_order))(*[int(x) for x in expert_order])
            if len(expert_order) != experts:
                raise ValueError("expert_order must name every expert once")
            d.expert_order = C.cast(keep, C.POINTER(C.c_uint32))
        d.format, d.backend, d.fused_transposed = fmt, backend, int(fused_transposed)
        return d, keep

    def layer_bytes(self, prefix: str, *, hidden: int, inter: int, experts: int, shared_inter: int = 0,
                    fmt: int = capi.CHECKPOINT_EXPERTS_BF16_FUSED, backend: int = capi.MOE_BACKEND_FUSED_BF16,
                    local=None, expert_order=None, fused_transposed: bool = False) -> tuple[int, int]:
        """``qs3_checkpoint_moe_layer_bytes``: validates the layer against the checkpoint and returns
        (weight bytes, load-time scratch bytes). No CUDA call."""
        d, _keep = self._layer_desc(prefix, hidden, inter, experts, shared_inter, fmt, backend, local, expert_order,
                                    fused_transposed)
        w, s = C.c_size_t(0), C.c_size_t(0)
        self.ctx.check(self._lib.qs3_checkpoint_moe_layer_bytes(self.ctx.handle, self.handle, C.byref(d),
                                                                C.byref(w), C.byref(s)))
        return int(w.value), int(s.value)


@dataclass
class LoadedMoeLayer:
    """Device tensors of one loaded layer (views into `block`), in the forms
    `ops.moe_layer_execute` takes."""
    block: "object"             # torch u8 tensor that owns the memory
    router: "object"            # bf16 [E, H]
    gate_up: "object"           # bf16 tensor or Nvfp4Weight
    down: "object"
    shared: SharedExpert | None
    act_global_scale: float
    act2_global_scale: float


def load_moe_layer(ckpt: Checkpoint, prefix: str, *, hidden: int, inter: int, experts: int, shared_inter: int = 0,
                   fmt: int = capi.CHECKPOINT_EXPERTS_BF16_FUSED, backend: int = capi.MOE_BACKEND_FUSED_BF16,
                   local=None, expert_order=None, fused_transposed: bool = False) -> LoadedMoeLayer:
    """``qs3_checkpoint_load_moe_layer`` into a freshly allocated device block."""
    import torch
    ctx = ckpt.ctx
    d, _keep = ckpt._layer_desc(prefix, hidden, inter, experts, shared_inter, fmt, backend, local, expert_order,
                                fused_transposed)
    wb, sb = C.c_size_t(0), C.c_size_t(0)
    ctx.check(ckpt._lib.qs3_checkpoint_moe_layer_bytes(ctx.handle, ckpt.handle, C.byref(d), C.byref(wb), C.byref(sb)))
    dev = torch.device("cuda", ctx.device)
    block = torch.empty(max(wb.value, 256), dtype=torch.uint8, device=dev)
    scratch = torch.empty(max(sb.value, 256), dtype=torch.uint8, device=dev)
    raw = capi.MoeLayerWeights()
    ctx.check(ckpt._lib.qs3_checkpoint_load_moe_layer(ctx.handle, ckpt.handle, C.byref(d), C.c_void_p(block.data_ptr()),
                                                      wb.value, C.c_void_p(scratch.data_ptr()), sb.value, C.byref(raw)))
    # the scratch block is released below: wait until the device passes that read it have run
    torch.cuda.synchronize(dev)
    base = block.data_ptr()
    torch_types = {capi.DTYPE_BF16: torch.bfloat16, capi.DTYPE_U8: torch.uint8, capi.DTYPE_F32: torch.float32}

    def view(t, rank):
        if not t.data:
            return None
        shape = [int(t.shape[i]) for i in range(rank)]
        dt = torch_types[t.dtype]
        n = int(np.prod(shape)) * torch.empty((), dtype=dt).element_size()
        off = t.data - base
        return block[off:off + n].view(dt).view(shape)

    nvfp4 = backend == capi.MOE_BACKEND_NVFP4

    def weight(w, sf, g):
        if not nvfp4:
            return view(w, 3)
        return Nvfp4Weight(packed=view(w, 3), scale_linear=None, scale_tiled=view(sf, 1), global_scale=view(g, 1))

    shared = None
    if shared_inter:
        shared = SharedExpert(weight(raw.shared_gate_up_weight, raw.shared_gate_up_scale_tiled,
                                     raw.shared_gate_up_global_scale),
                              weight(raw.shared_down_weight, raw.shared_down_scale_tiled, raw.shared_down_global_scale),
                              view(raw.shared_gate_weight, 2), shared_inter)
    return LoadedMoeLayer(block=block, router=view(raw.router_weight, 2),
                          gate_up=weight(raw.gate_up_weight, raw.gate_up_scale_tiled, raw.gate_up_global_scale),
                          down=weight(raw.down_weight, raw.down_scale_tiled, raw.down_global_scale),
                          shared=shared, act_global_scale=float(raw.act_global_scale),
                          act2_global_scale=float(raw.act2_global_scale))
