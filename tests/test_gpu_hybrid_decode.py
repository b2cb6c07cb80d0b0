"""The batched hybrid decode loop on a tiny configuration: every MoE block of a traced eager
step is checked against the CPU oracle (NVFP4 experts + shared expert, then the fused residual
add + next-layer RMSNorm), and the CUDA-graph replay of a step must reproduce the eager steps
token for token. The attention / GatedDeltaNet mixers are torch stand-ins and are not under
test; they only provide realistic inputs."""
import numpy as np
import pytest
import torch

from helpers import f32, max_abs, rel_l2, to_np

pytestmark = pytest.mark.gpu


def _triple(q):
    return to_np(q.packed), to_np(q.scale_linear), to_np(q.global_scale)


def test_moe_blocks_match_oracle_and_graph_matches_eager(oracle):
    from qs3_b200.hybrid_decode import HybridDecoder, tiny_config
    cfg = tiny_config(new_tokens=8)
    model = HybridDecoder(cfg, keep_linear_scales=True)
    start = model.snapshot()

    # ---- one traced eager step -------------------------------------------------------
    with torch.cuda.stream(model.stream):
        model.ctx.use_current_stream()
        model.trace = []
        model.step()
        model.stream.synchronize()
    trace, model.trace = model.trace, None
    assert model.ctx.read_device_error() == 0
    assert len(trace) == cfg.layers
    for layer, tr in enumerate(trace):
        blk = model.blocks[layer]
        normed = to_np(tr["normed"])
        ids, w = to_np(tr["ids"]), to_np(tr["weights"])
        # the routing of the traced step is the oracle's routing of the traced logits, bit for bit
        ids_ref, w_ref = oracle.router_topk(to_np(tr["logits"]), cfg.top_k, 0, True, 1.0)
        assert np.array_equal(ids, ids_ref)
        assert np.allclose(w, w_ref, atol=1e-5, rtol=0)
        hp, hs = oracle.nvfp4_quantize_act(normed, 1.0)
        moe = oracle.moe_nvfp4(hp, hs, ids, w, _triple(blk.gate_up), _triple(blk.down),
                               shared=dict(gu=_triple(blk.shared.gate_up), d=_triple(blk.shared.down),
                                           gate_w=to_np(blk.shared.gate_weight)),
                               hidden_bf16=normed)
        x_ref, res_ref = oracle.fused_add_rmsnorm(moe, to_np(tr["residual_in"]), to_np(model.input_norm[layer + 1]),
                                                  cfg.eps)
        # upstream's tolerances for the fused add + RMSNorm (tests_cuda_flashinfer_norm_rope.inc:1074-1258)
        # on top of the NVFP4 output tolerance of the block
        res = f32(to_np(tr["residual_out"]))
        assert np.max(np.abs(res - res_ref)) <= 0.012 + 2.0 ** -5 * np.max(np.abs(f32(moe)))
        x = f32(to_np(tr["x_out"]))
        assert np.linalg.norm(x - x_ref) / np.linalg.norm(x_ref) <= 1e-2
        assert np.max(np.abs(x - x_ref)) <= 0.018 + 2.0 ** -5 * np.max(np.abs(x_ref))

    # ---- eager steps vs graph replays from the same state ---------------------------------
    def run(n, graph=None):
        model.restore(start)
        toks = []
        with torch.cuda.stream(model.stream):
            model.ctx.use_current_stream()
            for _ in range(n):
                model.replay(graph) if graph is not None else model.step()
                toks.append(model.tokens.clone())
            model.stream.synchronize()
        return torch.stack(toks).cpu().numpy(), to_np(model.logits)

    eager_tokens, eager_logits = run(3)
    model.restore(start)
    graph = model.capture()
    graph_tokens, graph_logits = run(3, graph)
    assert model.ctx.read_device_error() == 0
    assert np.array_equal(eager_tokens, graph_tokens)
    assert np.array_equal(eager_logits, graph_logits)
    assert np.isfinite(f32(graph_logits)).all()
    assert int(model.pos.item()) == cfg.context + 3 == model.position
    # the host refuses to step past the cache instead of letting the device index out of range
    model.position = model.max_len
    with pytest.raises(RuntimeError, match="past the cache"):
        model.step()
    # the step really depends on its state: different tokens come out of successive steps
    assert not np.array_equal(eager_tokens[0], eager_tokens[1])


def test_library_only_graph_and_timing_helpers(oracle):
    """`time_steps` replays a graph with and without the mixers and leaves the decode state
    as it found it."""
    from qs3_b200.hybrid_decode import HybridDecoder, tiny_config
    cfg = tiny_config(new_tokens=8)
    model = HybridDecoder(cfg)
    before = [t.clone() for t, _ in model._state_tensors()]
    full = model.time_steps(3, mixers=True)
    lib = model.time_steps(3, mixers=False)
    assert full > 0 and lib > 0
    assert model.ctx.read_device_error() == 0
    for a, (b, _) in zip(before, model._state_tensors()):
        assert torch.equal(a, b)
    assert cfg.moe_weight_bytes_per_layer() == int((cfg.experts * 3 * cfg.inter * cfg.hidden
                                                    + 3 * cfg.shared_inter * cfg.hidden) * 9 / 16)


def test_paged_kv_cache_is_addressed_through_its_page_table():
    """Moving every page of the pool somewhere else and updating the page table accordingly must not
    change what the attention stand-in computes (bit for bit), and a step writes the new token's K / V
    into exactly one slot: page `kv_indices[kv_indptr[b] + pos // page_size]`, slot `pos % page_size`."""
    from qs3_b200.hybrid_decode import _Attention, tiny_config
    cfg = tiny_config(new_tokens=8, page_size=16)
    dev = torch.device("cuda", 0)
    max_len = cfg.context + cfg.new_tokens
    a = _Attention(cfg, torch.Generator(device=dev).manual_seed(1), dev, max_len)
    b = _Attention(cfg, torch.Generator(device=dev).manual_seed(1), dev, max_len)
    pages = a.k_pool.shape[0]
    assert a.kv_indptr.tolist() == [i * a.pages_per_seq for i in range(cfg.batch + 1)]
    assert sorted(a.kv_indices.tolist()) == list(range(pages)) and a.kv_indices.tolist() != list(range(pages))
    move = torch.randperm(pages, generator=torch.Generator(device=dev).manual_seed(2), device=dev)
    b.k_pool = torch.empty_like(a.k_pool).index_copy_(0, move, a.k_pool)     # page i now lives at move[i]
    b.v_pool = torch.empty_like(a.v_pool).index_copy_(0, move, a.v_pool)
    b.kv_indices = move[a.kv_indices.long()].to(torch.int32)
    slots = a.pages_per_seq * a.page
    mask = torch.full((1, 1, slots), float("-inf"), device=dev)
    mask[..., : cfg.context + 1] = 0.0
    x = (torch.randn((cfg.batch, cfg.hidden), device=dev) * 0.5).to(torch.bfloat16)
    pos = torch.full((1,), cfg.context, dtype=torch.long, device=dev)
    k_before = a.k_pool.clone()
    out_a, out_b = a(x, pos, mask), b(x, pos, mask)
    assert torch.equal(out_a, out_b)
    changed = (a.k_pool != k_before).flatten(1).any(dim=1).nonzero().flatten().tolist()
    table = a.kv_indices.view(cfg.batch, a.pages_per_seq)
    assert sorted(changed) == sorted(table[:, cfg.context // a.page].tolist())
    page0 = int(table[0, cfg.context // a.page])
    diff = (a.k_pool[page0] != k_before[page0]).any(dim=-1)                  # [kv_heads, page]
    assert diff[:, cfg.context % a.page].all() and int(diff.sum()) == cfg.kv_heads
