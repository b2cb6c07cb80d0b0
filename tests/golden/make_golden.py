"""Generates tests/golden/seeded_cases.npz: inputs-by-seed and CPU-oracle outputs of small seeded
MoE cases, so that (a) a change in the oracle shows up as a diff against committed vectors and
(b) the GPU tests have fixed vectors to hit that do not depend on the oracle being rebuilt.

    python tests/golden/make_golden.py

The upstream code is CUDA behind a Rust host and cannot be run or imported here, so these vectors
come from the CPU restatement (oracle/), whose own pins are the hand-transcribed upstream known
answers in reference_cases.json. Case "tiny_bf16" is the tiny bf16 configuration: 16 tokens, hidden
256, 8 experts, top-2 softmax router with renormalisation, intermediate 128, seed 0."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

CASES = {
    # name: (seed, tokens, hidden, experts, top_k, inter)
    "tiny_bf16": (0, 16, 256, 8, 2, 128),
    "small_bf16": (1, 48, 128, 16, 4, 64),
}


def build_case(oracle, helpers, seed, t, h, e, k, i):
    d = helpers.make_moe_inputs(seed, t, h, e, i)
    logits = oracle.gemm_bf16(d["hidden"], d["router"], "f32")
    ids, w = oracle.router_topk(logits, k, 0, True, 1.0)
    counts, indptr, route_rows, row_tokens, _ = oracle.route_sort(ids, w, 0, e)
    out = oracle.moe_bf16(d["hidden"], ids, w, d["gate_up"], d["down"])
    return dict(logits=logits, ids=ids, weights=w, counts=counts, indptr=indptr,
                route_rows=route_rows, row_tokens=row_tokens, out=out)


def main():
    from oracle import binding as oracle
    import helpers
    arrays = {}
    for name, (seed, t, h, e, k, i) in CASES.items():
        for key, val in build_case(oracle, helpers, seed, t, h, e, k, i).items():
            arrays[f"{name}/{key}"] = np.asarray(val)
    np.savez_compressed(os.path.join(HERE, "seeded_cases.npz"), **arrays)
    print("wrote", len(arrays), "arrays")


if __name__ == "__main__":
    main()
