"""Checked build (libqs3moe_checked.so, QSFI_ENABLE_CHECKED_VALIDATION=1): the device-side
input validators of upstream's checked test binary. Cases follow upstream
test_checked_moe_rejects_invalid_route_id / _non_finite_route_weight (test.cu:2168-2283) and the
router's non-finite check (tests_cuda_qscu_utils.inc:765-776); the release library accepts the
same inputs, as upstream's release binary does."""
import numpy as np
import pytest
import torch

from helpers import bf16, to_dev, to_np

pytestmark = pytest.mark.gpu
SENTINEL = 0xA5A5


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


@pytest.fixture(scope="module")
def checked(ops):
    return ops.capi.load_checked()


def _run_moe(ops, lib, route_id, route_weight):
    """One token, hidden 8, intermediate 8, two experts, top-1, all-zero weights."""
    ctx = ops.Context(lib=lib)
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=1, hidden_size=8, intermediate_size=8,
                                              num_experts=2, top_k=1))
    ws = torch.zeros(plan.workspace_size(1), dtype=torch.uint8, device="cuda")
    out = torch.from_numpy(np.full((1, 8), SENTINEL, np.uint16)).view(torch.bfloat16).cuda()
    zeros = lambda *shape: torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    ops.moe_execute_bf16(plan, zeros(1, 8), to_dev(np.array([[route_id]], np.int32)),
                         to_dev(np.array([[route_weight]], np.float32)), zeros(2, 16, 8), zeros(2, 8, 8), out, ws)
    torch.cuda.synchronize()
    return to_np(out)


@pytest.mark.parametrize("route_id,weight", [(2, 1.0), (1, float("nan")), (-1, 1.0), (0, float("inf"))])
def test_checked_moe_rejects_bad_routes(ops, checked, route_id, weight):
    with pytest.raises(ops.Qs3Error, match="MoE routes must target local experts and weights must be finite") as e:
        _run_moe(ops, checked, route_id, weight)
    assert e.value.status == ops.capi.STATUS_INVALID_ARGUMENT


def test_checked_moe_accepts_good_routes_and_release_skips_the_check(ops, checked):
    assert not _run_moe(ops, checked, 1, 0.5).any()            # zero weights: zero output, sentinel gone
    out = _run_moe(ops, ops.capi.load(), 2, 1.0)                # release: the stray route is ignored
    assert not out.any()


def test_checked_router_rejects_non_finite_logits(ops, checked):
    logits = np.array([[0.5, float("nan"), 1.0, -1.0]], np.float32)
    ids = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((1, 2), dtype=torch.float32, device="cuda")
    with pytest.raises(ops.Qs3Error) as e:
        ops.router_topk(to_dev(logits), ids, w, lib=checked)
    assert e.value.status == ops.capi.STATUS_INVALID_ARGUMENT
    ops.router_topk(to_dev(logits), ids, w)                     # release: NaN never wins a slot
    torch.cuda.synchronize()
    assert to_np(ids).tolist() == [[2, 0]]
    ops.router_topk(to_dev(np.nan_to_num(logits, nan=-3.0)), ids, w, lib=checked)   # finite: accepted
    torch.cuda.synchronize()
    assert to_np(ids).tolist() == [[2, 0]]


def test_checked_expert_parallel_plan_accepts_remote_routes(ops, checked):
    """A plan that owns only part of the experts sees routes to the other ranks' experts."""
    ctx = ops.Context(lib=checked)
    plan = ops.MoePlan(ctx, ops.MoePlanConfig(max_num_tokens=2, hidden_size=8, intermediate_size=8,
                                              num_experts=4, top_k=2, local_expert_offset=2,
                                              local_num_experts=2))
    ws = torch.zeros(plan.workspace_size(2), dtype=torch.uint8, device="cuda")
    out = torch.zeros((2, 8), dtype=torch.bfloat16, device="cuda")
    zeros = lambda *shape: torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
    ids = to_dev(np.array([[0, 3], [2, 1]], np.int32))
    w = to_dev(np.full((2, 2), 0.5, np.float32))
    ops.moe_execute_bf16(plan, zeros(2, 8), ids, w, zeros(2, 16, 8), zeros(2, 8, 8), out, ws)
    with pytest.raises(ops.Qs3Error, match="MoE routes must target"):
        ops.moe_execute_bf16(plan, zeros(2, 8), to_dev(np.array([[0, 4], [2, 1]], np.int32)), w,
                             zeros(2, 16, 8), zeros(2, 8, 8), out, ws)
