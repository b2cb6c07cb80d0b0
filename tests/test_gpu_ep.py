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


def test_route_targets_and_routed_pull_on_one_gpu():
    """The de-duplicated dispatch without a second GPU: two ranks' token blocks live side by side on this
    device. `qs3_moe_ep_route` must report, per token, the set of ranks it has a route to (and the slot
    ids of a placement with replicated experts), and `qs3_moe_ep_pull_routed` must copy ids and weights of
    every token but codes and scales only of the tokens routed to the pulling rank."""
    from qs3_b200 import ep, ops, workload
    ctx = ops.Context(0)
    world, per, hot = 2, 8, [3, 12]
    cfg = workload.LayerConfig("ep_pull", 200, 512, 16, 4, 256, 0, True, 1.1)
    t, h, k = cfg.tokens, cfg.hidden, cfg.top_k
    blocks, wants = [], []
    seg_sizes = [t * (h // 2), t * (h // 16), t * k * 4, t * k * 4, t * 4]
    offs, total = [], 0
    for sz in seg_sizes:
        offs.append(total)
        total += (sz + 255) // 256 * 256
    for rank in range(world):
        data = workload.LayerData(cfg, ctx, seed=6, expert_range=(rank * per, per), token_seed=rank + 1,
                                  hot_positions=hot)
        backend = ep.CudaBackend(ctx, data, world)
        assert backend.slot_range == (rank * (per + 2), per + 2)
        block = torch.zeros(total, dtype=torch.uint8, device="cuda")
        seg = lambda j, dt, shape: block[offs[j]:offs[j] + seg_sizes[j]].view(dt).view(shape)
        backend.bind_route_outputs(seg(0, torch.uint8, (t, h // 2)), seg(1, torch.uint8, (t, h // 16)),
                                   seg(2, torch.int32, (t, k)), seg(3, torch.float32, (t, k)),
                                   seg(4, torch.int32, (t,)))
        backend.route(data.hidden)
        torch.cuda.synchronize()
        ids = backend.ids.cpu().numpy()
        table = np.array(ep.slot_id_table(cfg.experts, world, hot, rank))
        slots = table[ids]
        assert np.array_equal(backend.dispatch_ids.cpu().numpy(), slots)
        mask = np.zeros(t, np.int64)
        for r in range(world):
            mask |= ((slots // (per + 2)) == r).any(axis=1).astype(np.int64) << r
        assert np.array_equal(backend.mask.cpu().numpy().astype(np.int64), mask)
        assert (mask & (1 << rank)).all() or not np.isin(ids, hot).any(axis=1).all()
        blocks.append(block)
        wants.append(mask)
        last = backend
    for me in range(world):
        sentinel = 0xA5
        g_codes = torch.full((world * t, h // 2), sentinel, dtype=torch.uint8, device="cuda")
        g_scale = torch.full((world * t, h // 16), sentinel, dtype=torch.uint8, device="cuda")
        g_ids = torch.full((world * t, k), -7, dtype=torch.int32, device="cuda")
        g_wts = torch.full((world * t, k), -7.0, dtype=torch.float32, device="cuda")
        last.rank = me
        last.pull_routed([b.data_ptr() for b in blocks], offs, (g_codes, g_scale, g_ids, g_wts))
        torch.cuda.synchronize()
        for r in range(world):
            seg = lambda j, dt, shape: blocks[r][offs[j]:offs[j] + seg_sizes[j]].view(dt).view(shape)
            rows = slice(r * t, (r + 1) * t)
            assert torch.equal(g_ids[rows], seg(2, torch.int32, (t, k)))
            assert torch.equal(g_wts[rows], seg(3, torch.float32, (t, k)))
            wanted = torch.from_numpy(((wants[r] >> me) & 1).astype(bool)).cuda()
            assert 0 < int(wanted.sum()) < t or r == me
            assert torch.equal(g_codes[rows][wanted], seg(0, torch.uint8, (t, h // 2))[wanted])
            assert torch.equal(g_scale[rows][wanted], seg(1, torch.uint8, (t, h // 16))[wanted])
            assert bool((g_codes[rows][~wanted] == sentinel).all()) and bool((g_scale[rows][~wanted] == sentinel).all())
    assert ctx.read_device_error() == 0
