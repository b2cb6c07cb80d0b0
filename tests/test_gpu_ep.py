"""Expert-parallel compute phases on one GPU (world size 1, NCCL): route -> local experts
-> finish must reproduce the single-call layer, and a split of the experts over two
plans on the same GPU must sum to the full result (what two ranks would exchange)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist

from helpers import f32, rel_l2, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def group():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    yield
    dist.destroy_process_group()


def test_world_size_one_equals_the_layer_call(group):
    from qs3_b200 import ep, ops, workload
    ctx = ops.Context(0)
    cfg = workload.LayerConfig("ep_small", 300, 512, 32, 4, 256, 256, True, 1.1)
    data = workload.LayerData(cfg, ctx, seed=3)
    layer = ep.ExpertParallelLayer(ctx, data, 0, 1)
    out_ep = to_np(layer.step())
    out_ep2 = to_np(layer.step())
    torch.cuda.synchronize()
    assert np.array_equal(out_ep, out_ep2)
    plan = data.plan(ctx)
    ws = torch.empty(plan.layer_workspace_size(cfg.tokens, cfg.shared_inter), dtype=torch.uint8, device="cuda")
    out = torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    ids = torch.empty((cfg.tokens, cfg.top_k), dtype=torch.int32, device="cuda")
    ops.moe_layer_execute(plan, data.hidden, data.router, data.gate_up, data.down, out, ws,
                          router_bias=data.bias, shared=data.shared, topk_ids=ids)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    assert np.array_equal(to_np(ids), to_np(layer.backend.ids))          # routing: bit-exact
    # the EP path rounds the routed sum to bf16 once more before adding the shared term
    assert rel_l2(out_ep, to_np(out)) <= 4e-3
    assert np.max(np.abs(f32(out_ep) - f32(to_np(out)))) <= 2.0 ** -6 * np.max(np.abs(f32(to_np(out))))


def test_two_expert_blocks_sum_to_the_full_result(group):
    """Both halves of the experts on one GPU: their partial sums are what two ranks exchange."""
    from qs3_b200 import ep, ops, workload
    ctx = ops.Context(0)
    cfg = workload.LayerConfig("ep_small", 200, 512, 16, 4, 256, 0, True, 0.0)
    full = workload.LayerData(cfg, ctx, seed=4)
    ref = to_np(ep.ExpertParallelLayer(ctx, full, 0, 1).step()).copy()
    total = np.zeros(ref.shape, np.float64)
    for r in range(2):
        first, count = ep.expert_block(r, 2, cfg.experts)
        part = workload.LayerData(cfg, ctx, seed=4, expert_range=(first, count))
        layer = ep.ExpertParallelLayer(ctx, part, 0, 1)
        total += f32(to_np(layer.step()))
    torch.cuda.synchronize()
    want = f32(ref).astype(np.float64)
    assert np.linalg.norm(total - want) <= 1e-2 * np.linalg.norm(want)
