"""GPU test of ``qs3_moe_route_sort_static``, the route sort for callers that cannot
allocate device memory (its scratch is a fixed array inside the library).

The file name sorts last on purpose: a run that stops at the first failure has then
already executed every other test. The test is self-contained, so it also passes alone
in a fresh process (where its first call is the one that resolves the scratch address).

It calls the entry point through the C ABI twice in a row, with different problem sizes,
and requires each result to be bit-identical (integer tables and the copied f32 weights)
to what the existing path reports for the same routing: ``qsfi_moe_execute_bf16``
followed by ``qs3_moe_routing_tables``. The second, smaller call would expose stale
scratch contents from the first.
"""
import numpy as np
import pytest
import torch

from helpers import to_dev, to_np

pytestmark = pytest.mark.gpu


def _existing_tables(ops, ctx, ids_np, w_np, experts, local_offset, local_experts):
    """Routing tables from the existing entry points (scratch in a caller workspace)."""
    t, k = ids_np.shape
    h = i = 8
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=t, hidden_size=h, intermediate_size=i,
                                              num_experts=experts, top_k=k,
                                              local_expert_offset=local_offset,
                                              local_num_experts=local_experts))
    ws = torch.zeros(plan.workspace_size(t), dtype=torch.uint8, device="cuda")
    z = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device="cuda")
    ops.moe_execute_bf16(plan, z(t, h), to_dev(ids_np), to_dev(w_np), z(local_experts, 2 * i, h),
                         z(local_experts, h, i), z(t, h), ws)
    return [to_np(x) for x in plan.routing_tables(ws, t)]


def test_static_route_sort_matches_existing_path_twice_in_a_row():
    from qs3_b200 import capi, ops
    ctx = ops.Context()
    rng = np.random.default_rng(2024)
    # two different problems back to back: a large skewed one, then a small expert-parallel one
    problems = [dict(t=3000, k=10, e=512, off=0, le=512), dict(t=77, k=4, e=64, off=16, le=24)]
    prepared = []
    for p in problems:
        ids = np.minimum((rng.pareto(0.9, size=(p["t"], p["k"])) * 5).astype(np.int64), p["e"] - 1).astype(np.int32)
        ids[0, :] = ids[0, 0]  # duplicated routes inside one token
        w = rng.random((p["t"], p["k"]), dtype=np.float32)
        prepared.append((p, ids, w, _existing_tables(ops, ctx, ids, w, p["e"], p["off"], p["le"])))

    for p, ids, w, want in prepared:  # the two calls under test, nothing in between
        got = ops.route_sort_static(ctx, to_dev(ids), to_dev(w), p["off"], p["le"])
        torch.cuda.synchronize()
        counts, indptr, route_rows, row_tokens, row_scales = (to_np(x) for x in got)
        n = int(indptr[-1])
        assert np.array_equal(counts, want[0])
        assert np.array_equal(indptr, want[1])
        assert np.array_equal(route_rows, want[2])
        assert np.array_equal(row_tokens[:n], want[3])
        assert np.array_equal(row_scales[:n], want[4])  # copied weights: bit-exact

    # beyond the fixed scratch: a clear refusal, no launch
    big = torch.zeros((capi.ROUTE_SORT_STATIC_MAX_ROUTES // 8 + 1, 8), dtype=torch.int32, device="cuda")
    with pytest.raises(ops.Qs3Error) as e:
        ops.route_sort_static(ctx, big, big.float(), 0, 8)
    assert e.value.status == capi.STATUS_UNSUPPORTED and "at most 131072 routes" in e.value.message
    with pytest.raises(ops.Qs3Error) as e:
        ops.route_sort_static(ctx, big[:4], big[:4].float(), 0, capi.ROUTE_SORT_STATIC_MAX_EXPERTS + 1)
    assert e.value.status == capi.STATUS_UNSUPPORTED and "1024 local experts" in e.value.message


def test_static_route_sort_small_path_allocates_nothing():
    """At most 1024 routes take the fused single-block kernel; then a larger problem follows, both
    with caller-created outputs. Device memory as the driver reports it (free bytes) and as torch's
    caching allocator holds it (reserved bytes) must not move across the calls: the entry point's
    scratch lives inside the library and neither it nor the wrapper may allocate."""
    from qs3_b200 import ops
    ctx = ops.Context()
    rng = np.random.default_rng(7)
    problems = [dict(t=100, k=8, e=32, off=0, le=32), dict(t=2000, k=10, e=256, off=64, le=128)]
    prepared = []
    for p in problems:
        ids = rng.integers(0, p["e"], size=(p["t"], p["k"]), dtype=np.int32)
        w = rng.random((p["t"], p["k"]), dtype=np.float32)
        want = _existing_tables(ops, ctx, ids, w, p["e"], p["off"], p["le"])
        r = p["t"] * p["k"]
        i32 = lambda n: torch.full((n,), -7, dtype=torch.int32, device="cuda")
        out = (i32(p["le"]), i32(p["le"] + 1), i32(r), i32(r), torch.zeros(r, dtype=torch.float32, device="cuda"))
        prepared.append((p, to_dev(ids), to_dev(w), want, out))
    # the first call on a device resolves the scratch address (a symbol lookup, not an allocation);
    # do it before the measurement so that the window below holds steady-state calls only
    p, ids, w, _, out = prepared[0]
    ops.route_sort_static(ctx, ids, w, p["off"], p["le"], out=out)
    torch.cuda.synchronize()

    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for p, ids, w, _, out in prepared:
        ops.route_sort_static(ctx, ids, w, p["off"], p["le"], out=out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_reserved() == reserved_before
    assert free_after == free_before

    for p, _, _, want, out in prepared:
        counts, indptr, route_rows, row_tokens, row_scales = (to_np(x) for x in out)
        n = int(indptr[-1])
        assert np.array_equal(counts, want[0])
        assert np.array_equal(indptr, want[1])
        assert np.array_equal(route_rows, want[2])
        assert np.array_equal(row_tokens[:n], want[3])
        assert np.array_equal(row_scales[:n], want[4])
