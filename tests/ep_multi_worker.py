"""Child process of tests/test_gpu_ep_multi.py: one rank of an expert-parallel layer on
its own GPU. Each rank also holds ALL experts (small configuration) and computes the
single-GPU result for its tokens through qs3_moe_layer_execute; the expert-parallel
result must match it (routing bit-exact, output within the bf16 tolerance)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from helpers import f32, to_np
    from qs3_b200 import ep, ops, workload
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = ops.Context(local)
    cfg = workload.LayerConfig("ep_multi", 512, 512, 32, 4, 256, 256, True, 1.1)
    first, count = ep.expert_block(rank, world, cfg.experts)
    balance = world if os.environ.get("QS3_TEST_BALANCED") == "1" else 0
    hot = int(os.environ.get("QS3_TEST_HOT", "0")) if balance else 0
    part = workload.LayerData(cfg, ctx, seed=9, expert_range=(first, count), token_seed=rank + 1,
                              balance_world=balance, hot_experts=hot)
    assert len(part.hot_positions) == hot
    layer = ep.ExpertParallelLayer(ctx, part, rank, world)
    for _ in range(3):
        out = layer.step()
    torch.cuda.synchronize()
    got = to_np(out)

    full = workload.LayerData(cfg, ctx, seed=9, token_seed=rank + 1, placement=part.placement)
    assert torch.equal(full.hidden, part.hidden)
    assert torch.equal(full.router, part.router)
    if balance:
        assert part.placement != list(range(cfg.experts))
    plan = full.plan(ctx)
    ws = torch.empty(plan.layer_workspace_size(cfg.tokens, cfg.shared_inter), dtype=torch.uint8, device="cuda")
    ref = torch.empty((cfg.tokens, cfg.hidden), dtype=torch.bfloat16, device="cuda")
    ids = torch.empty((cfg.tokens, cfg.top_k), dtype=torch.int32, device="cuda")
    ops.moe_layer_execute(plan, full.hidden, full.router, full.gate_up, full.down, ref, ws,
                          router_bias=full.bias, shared=full.shared, topk_ids=ids)
    torch.cuda.synchronize()
    assert ctx.read_device_error() == 0
    assert torch.equal(ids, layer.backend.ids), "routing differs between EP and single-GPU"
    want = f32(to_np(ref)).astype(np.float64)
    err = np.linalg.norm(f32(got) - want) / np.linalg.norm(want)
    assert err <= 1e-2, err
    assert np.max(np.abs(f32(got) - want)) <= 2.0 ** -5 * np.max(np.abs(want))
    # the same step replayed from a CUDA graph (barrier epochs counted on the device): bit-identical
    layer.try_capture()
    graphed = layer.graph is not None
    if layer.combine_mode == "pull" and layer.dispatch_mode == "pull":
        assert graphed, "the peer-load step must be capturable"
        for _ in range(3):
            replayed = layer.step()
        torch.cuda.synchronize()
        layer.check()
        assert np.array_equal(to_np(replayed), got), "graph replay differs from eager launches"
    dist.barrier()
    if rank == 0:
        print(f"EP_MULTI_OK world={world} rel_l2={err:.3e} combine={layer.combine_mode} balanced={bool(balance)} "
              f"hot={hot} graph={graphed}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
