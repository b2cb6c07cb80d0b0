"""The reference's own GPU BF16 MoE path (`qsfi_context.cu`, `qsfi_moe.cu`, `qscu.cu`), compiled from
the sources where they lie, as an A/B oracle for the BF16 chain at sizes the reference's own tests
(two tokens) do not reach. Test infrastructure only.

``build()`` runs the recipe: the reference's macro generator (`build_tools/generate_macros.c`, plain C)
is compiled and run to produce `qsfi_macros.h`, then nvcc compiles a two-line translation unit that
includes the two qsfi files, plus `qscu.cu`, for sm_100a against the FlashInfer / CUTLASS headers of
the installed `flashinfer` Python package (the reference's own `3pty/flashinfer` submodule is empty and
its pin unrecorded, so this is a stand-in revision: good for an A/B check, not a source to port).
Everything is written to ``oracle/_ref/`` (git-ignored); no reference source is copied. The recipe needs
the reference tree (its directory is ``REF_DIR`` below, overridable with ``QS3_REFERENCE_DIR``); machines
without it use the
prebuilt ``oracle/_ref/libqs3ref.so`` if present.

``load()`` binds the upstream subset of the C ABI with the ctypes structures of ``qs3_b200.capi`` (the
layouts are the same by construction), so ``qs3_b200.ops`` wrappers run on it with ``lib=``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("QS3_REFERENCE_DIR", "/root/reference")
OUT_DIR = os.path.join(_HERE, "_ref")
LIB_PATH = os.path.join(OUT_DIR, "libqs3ref.so")

UPSTREAM_SYMBOLS = (
    "qsfi_context_create", "qsfi_context_destroy", "qsfi_context_get_last_error", "qsfi_context_set_stream",
    "qsfi_moe_plan_create", "qsfi_moe_plan_destroy", "qsfi_moe_workspace_size", "qsfi_moe_execute_bf16",
    "qscu_router_topk", "qscu_silu_and_mul_bf16", "qscu_qwen36_shared_expert_gate_add_bf16",
)


def available() -> bool:
    return os.path.exists(LIB_PATH)


def build(force: bool = False) -> str | None:
    """Compile the reference path into ``oracle/_ref/libqs3ref.so``; returns the path, or None when the
    reference tree or the FlashInfer headers are not on this machine (the prebuilt file is then used)."""
    sources = [os.path.join(REF_DIR, f) for f in ("qsfi_context.cu", "qsfi_moe.cu", "qscu.cu")]
    if not all(os.path.exists(s) for s in sources):
        return LIB_PATH if available() else None
    if available() and not force and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in sources):
        return LIB_PATH
    try:
        import flashinfer
    except Exception:
        return LIB_PATH if available() else None
    data = os.path.join(os.path.dirname(flashinfer.__file__), "data")
    os.makedirs(OUT_DIR, exist_ok=True)
    gen = os.path.join(OUT_DIR, "gen_macros")
    subprocess.run(["gcc", "-O1", "-o", gen, os.path.join(REF_DIR, "build_tools", "generate_macros.c")], check=True)
    with open(os.path.join(OUT_DIR, "qsfi_macros.h"), "w") as f:
        subprocess.run([gen], check=True, stdout=f)
    tu = os.path.join(OUT_DIR, "ref_tu.cu")
    with open(tu, "w") as f:
        f.write('#include "qsfi_context.cu"\n#include "qsfi_moe.cu"\n')
    includes = [OUT_DIR, REF_DIR, os.path.join(data, "include"), os.path.join(data, "cutlass", "include"),
                os.path.join(data, "cutlass", "tools", "util", "include"), os.path.join(data, "spdlog", "include"),
                os.path.join(data, "csrc")]
    cmd = ["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr", "-O2",
           "-Xcompiler", "-fPIC", "-shared", "-diag-suppress", "20012"]
    for inc in includes:
        cmd += ["-I", inc]
    cmd += [tu, os.path.join(REF_DIR, "qscu.cu"), "-o", LIB_PATH]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(os.path.join(OUT_DIR, "build.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("reference build failed, see oracle/_ref/build.log:\n" + r.stderr[-2000:])
    return LIB_PATH


def load() -> C.CDLL:
    from qs3_b200 import capi
    lib = C.CDLL(LIB_PATH)
    for name in UPSTREAM_SYMBOLS:
        res, args = capi._SIGNATURES[name]
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def workspace_tables(workspace, num_tokens: int, top_k: int, local_experts: int):
    """counts, indptr, route_rows, row_tokens of the reference's last execute, read out of its
    workspace (layout of compute_workspace_layout, qsfi_moe.cu:67-121: counts[E], indptr[E+1],
    write_offsets[E], route_rows[R], row_tokens[R], ... each 256-byte aligned)."""
    import torch
    r = num_tokens * top_k
    sizes = [local_experts * 4, (local_experts + 1) * 4, local_experts * 4, r * 4, r * 4]
    offs, off = [], 0
    for sz in sizes:
        off = (off + 255) // 256 * 256
        offs.append(off)
        off += sz
    grab = lambda j, n: workspace[offs[j]:offs[j] + 4 * n].view(torch.int32).cpu().numpy().copy()
    counts, indptr = grab(0, local_experts), grab(1, local_experts + 1)
    return counts, indptr, grab(3, r), grab(4, r)[: int(indptr[-1])]


if __name__ == "__main__":
    print(build(force=True))
