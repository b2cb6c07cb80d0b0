"""qs3_b200 -- the qs3 mixture-of-experts layer as hand-written sm_100a CUDA behind
qs3's C ABI, plus the thin host layer (ctypes + torch device tensors) that tests,
the benchmark and the expert-parallel driver use.

Nothing here falls back to a CPU or library implementation: importing
:mod:`qs3_b200.ops` and calling an operator requires ``libqs3moe.so`` (built by
``python -m qs3_b200._build``) and a B200.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
