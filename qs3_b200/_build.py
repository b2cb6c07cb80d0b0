"""In-tree build of ``libqs3moe.so`` (CUDA, sm_100a only).

``python -m qs3_b200._build`` compiles every translation unit under
``qs3_b200/csrc`` with nvcc for ``sm_100a`` and links them into
``qs3_b200/libqs3moe.so``. nvcc cross-compiles without a GPU, so this also runs
on a CPU-only machine; the shared object is what a GPU machine loads.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(SRC_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libqs3moe.so")
CHECKED_LIB_PATH = os.path.join(PKG_DIR, "libqs3moe_checked.so")

SOURCES = ["context.cu", "router.cu", "routing.cu", "gemm.cu", "gemm_api.cu", "nvfp4.cu", "moe.cu",
           "peak_probe.cu", "fp8.cu", "norm.cu", "loader.cu", "nvfp4_decode.cu", "gemm_dense.cu", "gemm_pair.cu", "failure.cu"]
HEADERS = ["common.cuh", "nvfp4.cuh", "tcgen05.cuh", os.path.join("..", "..", "include", "qs3_moe.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """Compile the library in-tree. ``checked`` builds the variant with device-side input
    validation (``-DQSFI_ENABLE_CHECKED_VALIDATION=1``, as upstream's checked test binary):
    ``libqs3moe_checked.so`` next to the release ``libqs3moe.so``."""
    nvcc = _nvcc()
    obj_dir = OBJ_DIR + ("_checked" if checked else "")
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    flags = NVCC_FLAGS + (["-DQSFI_ENABLE_CHECKED_VALIDATION=1"] if checked else [])
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(SRC_DIR, h) for h in HEADERS]
    jobs = []
    for src in SOURCES:
        s = os.path.join(SRC_DIR, src)
        o = os.path.join(obj_dir, src.replace(".cu", ".o"))
        if force or _stale(o, [s] + headers):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *flags, "-c", s, "-o", o]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return s, r

    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for s, r in pool.map(compile_one, jobs):
            if verbose and r.stderr:
                sys.stderr.write(r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {s}:\n{r.stdout}\n{r.stderr}")
    objs = [os.path.join(obj_dir, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(lib_path, objs):
        cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked=True))
