"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2 and 4).

The product's compute phases need a GPU, so these tests plug a CPU stand-in backend
(built on the oracle) into ``qs3_b200.ep.ExpertParallelLayer`` and check what the
host-side logic is responsible for: the expert partition, the layout of the gathered
token buffers, the direction of the partial-sum all-to-all and the rank-ordered
summation. The n-rank result must equal the single-rank oracle result of the same
global batch.
"""
import os
import socket
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

CFG = SimpleNamespace(tokens=24, hidden=256, experts=8, top_k=3, inter=256, shared_inter=256, nvfp4=True)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def _np16(t):
    return t.contiguous().view(torch.uint16).numpy()


def _weights(orc):
    """Quantised weights shared by every rank (seeded), as oracle triples."""
    from helpers import make_moe_inputs
    d = make_moe_inputs(5, 4, CFG.hidden, CFG.experts, CFG.inter, CFG.shared_inter)
    q = lambda w, gated: tuple(np.asarray(x) for x in (lambda r: (r[0], r[1], r[3]))(orc.nvfp4_quantize_weight(w, gated)))
    return dict(router=d["router"], gu=q(d["gate_up"], True), d=q(d["down"], False),
                sgu=q(d["sh_gate_up"], True), sd=q(d["sh_down"], False), sgate=d["sh_gate"])


def _tokens(rank):
    from helpers import bf16
    rng = np.random.default_rng(100 + rank)
    return bf16(rng.standard_normal((CFG.tokens, CFG.hidden), dtype=np.float32))


class OracleBackend:
    """CPU stand-in for ``qs3_b200.ep.CudaBackend`` (same four methods)."""

    def __init__(self, orc, w, first, count, world):
        self.orc, self.w, self.first, self.count, self.world = orc, w, first, count, world
        self.shared_out = None

    def route(self, hidden):
        hid = _np16(hidden)
        ids, wts = self.orc.router_topk(self.orc.gemm_bf16(hid, self.w["router"], "f32"), CFG.top_k, 0, True, 1.0)
        packed, scale = self.orc.nvfp4_quantize_act(hid, 1.0)
        return (torch.from_numpy(packed), torch.from_numpy(scale), torch.from_numpy(ids), torch.from_numpy(wts))

    def experts(self, packed, scale, ids, wts, out):
        sl = slice(self.first, self.first + self.count)
        gu = tuple(x[sl] for x in self.w["gu"])
        dn = tuple(x[sl] for x in self.w["d"])
        res = self.orc.moe_nvfp4(packed.numpy(), scale.numpy(), ids.numpy(), wts.numpy(), gu, dn,
                                 local_offset=self.first)
        out.copy_(_bf(res))

    def shared_expert(self, hidden):
        self.hidden = hidden

    def finish(self, hidden, partials, out):
        hid = _np16(hidden)
        t = hid.shape[0]
        hp, hs = self.orc.nvfp4_quantize_act(hid, 1.0)
        # shared expert alone: no routed experts (an id outside every local range)
        none_ids = np.full((t, 1), -1, np.int32)
        sh = self.orc.moe_nvfp4(hp, hs, none_ids, np.zeros((t, 1), np.float32), self.w["gu"], self.w["d"],
                                shared=dict(gu=self.w["sgu"], d=self.w["sd"], gate_w=self.w["sgate"]),
                                hidden_bf16=hid)
        acc = self.orc.bf16_to_f32(sh).astype(np.float32)
        for r in range(self.world):
            acc = acc + self.orc.bf16_to_f32(_np16(partials[r]))
        out.copy_(_bf(self.orc.f32_to_bf16(acc)))


class ReplicatedOracleBackend(OracleBackend):
    """As above with the experts in ``hot`` replicated on every rank: the rank's slots are its own
    experts followed by the replicas, and routes travel as slot ids (``ep.slot_id_table``)."""

    def __init__(self, orc, w, first, count, world, hot):
        super().__init__(orc, w, first, count, world)
        from qs3_b200 import ep
        self.rank = first // count
        self.slots = count + len(hot)
        self.table = np.array(ep.slot_id_table(CFG.experts, world, hot, self.rank), np.int32)
        local = list(range(first, first + count)) + list(hot)
        self.gu = tuple(x[local] for x in w["gu"])
        self.dn = tuple(x[local] for x in w["d"])

    def route(self, hidden):
        packed, scale, ids, wts = super().route(hidden)
        self.ids = ids
        return packed, scale, torch.from_numpy(self.table[ids.numpy()]), wts

    def experts(self, packed, scale, ids, wts, out):
        res = self.orc.moe_nvfp4(packed.numpy(), scale.numpy(), ids.numpy(), wts.numpy(), self.gu, self.dn,
                                 local_offset=self.rank * self.slots)
        out.copy_(_bf(res))


def _worker(rank, world, port, results, hot=()):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import binding as orc
        from qs3_b200 import ep
        w = _weights(orc)
        first, count = ep.expert_block(rank, world, CFG.experts)
        data = SimpleNamespace(cfg=CFG, hidden=_bf(_tokens(rank)), expert_range=(first, count), shared=True)
        backend = (ReplicatedOracleBackend(orc, w, first, count, world, list(hot)) if hot
                   else OracleBackend(orc, w, first, count, world))
        layer = ep.ExpertParallelLayer(None, data, rank, world, backend=backend)
        out1 = _np16(layer.step()).copy()
        out2 = _np16(layer.step()).copy()  # buffers are reused: a second step must give the same answer
        assert np.array_equal(out1, out2)
        # gathered layout: rank r's tokens sit in rows [r*T, (r+1)*T)
        mine = slice(rank * CFG.tokens, (rank + 1) * CFG.tokens)
        hp, _ = orc.nvfp4_quantize_act(_tokens(rank), 1.0)
        assert np.array_equal(layer.g_packed[mine].numpy(), hp)
        results[rank] = out1
    finally:
        dist.destroy_process_group()


def _single_rank_reference(orc, world):
    w = _weights(orc)
    outs = []
    for rank in range(world):
        hid = _tokens(rank)
        ids, wts = orc.router_topk(orc.gemm_bf16(hid, w["router"], "f32"), CFG.top_k, 0, True, 1.0)
        hp, hs = orc.nvfp4_quantize_act(hid, 1.0)
        outs.append(orc.moe_nvfp4(hp, hs, ids, wts, w["gu"], w["d"],
                                  shared=dict(gu=w["sgu"], d=w["sd"], gate_w=w["sgate"]), hidden_bf16=hid))
    return outs


@pytest.mark.parametrize("world,hot", [(2, ()), (4, ()), (2, (5, 0)), (4, (6, 3, 1))])
def test_expert_parallel_equals_single_rank(oracle, world, hot):
    """`hot`: experts replicated on every rank; their routes are served by the token's own rank."""
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, port, results, hot), nprocs=world, join=True)
    ref = _single_rank_reference(oracle, world)
    for rank in range(world):
        got = oracle.bf16_to_f32(results[rank]).astype(np.float64)
        want = oracle.bf16_to_f32(ref[rank]).astype(np.float64)
        # partial sums are rounded to bf16 per rank before the ordered sum: not bit-exact by design
        assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
        assert np.max(np.abs(got - want)) <= 2.0 ** -5 * np.max(np.abs(want))


def _failing_worker(rank, world, port, results):
    """Rank 1 fails between steps (host side: it raises before its second dispatch and leaves);
    rank 0 must get an error from its own step within the process group's timeout, not hang."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    try:
        from oracle import binding as orc
        from qs3_b200 import ep, ops
        w = _weights(orc)
        first, count = ep.expert_block(rank, world, CFG.experts)
        data = SimpleNamespace(cfg=CFG, hidden=_bf(_tokens(rank)), expert_range=(first, count), shared=True)
        layer = ep.ExpertParallelLayer(None, data, rank, world, backend=OracleBackend(orc, w, first, count, world))
        layer.step()                                   # a healthy step first
        if rank == 1:
            results[rank] = "left"
            return                                     # the failure: this rank never dispatches again
        t0 = time.perf_counter()
        try:
            layer.step()
            results[rank] = "no error"
        except ops.Qs3Error as exc:
            results[rank] = ("error", exc.status, time.perf_counter() - t0)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_rank_that_leaves_between_steps_is_reported_not_waited_for():
    port = _free_port()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_failing_worker, args=(2, port, results), nprocs=2, join=True)
    assert results[1] == "left"
    kind, status, seconds = results[0]
    from qs3_b200 import capi
    assert kind == "error" and status == capi.STATUS_BACKEND_ERROR
    assert seconds < 30


def test_slot_table_of_a_replicated_placement():
    from qs3_b200.ep import hottest_experts, slot_id_table
    counts = [5, 90, 7, 80, 3, 80, 1, 2]
    assert hottest_experts(counts, 3) == [1, 3, 5]           # descending count, ties by id
    world, hot = 2, [1, 5]
    per, slots = 4, 6
    for rank in range(world):
        table = slot_id_table(8, world, hot, rank)
        for e, slot in enumerate(table):
            holder, index = divmod(slot, slots)
            if e in hot:
                assert holder == rank and index == per + hot.index(e)   # served where the token lives
            else:
                assert holder == e // per and index == e % per           # served by the owner
        assert len(set(table)) == 8


def test_expert_block_partition():
    from qs3_b200 import ep
    assert [ep.expert_block(r, 4, 512) for r in range(4)] == [(0, 128), (128, 128), (256, 128), (384, 128)]
    with pytest.raises(ValueError):
        ep.expert_block(0, 3, 512)


def test_balanced_placement_evens_rank_loads():
    """Static placement from routing statistics: a permutation with equal expert counts per
    rank whose per-rank load is far more even than contiguous blocks under a skewed load."""
    from qs3_b200.ep import balanced_placement
    rng = np.random.default_rng(3)
    counts = (40000.0 / (1.0 + rng.permutation(64)) ** 1.1).astype(np.int64)
    for world in (2, 4, 8):
        place = balanced_placement(counts, world)
        assert sorted(place) == list(range(64))
        per = 64 // world
        loads = [int(counts[place[r * per:(r + 1) * per]].sum()) for r in range(world)]
        blocks = [int(counts[r * per:(r + 1) * per].sum()) for r in range(world)]
        assert max(loads) <= max(blocks)
        # as even as equal expert counts allow: the rank of the hottest expert also has to
        # take per - 1 others, at best the coldest ones
        floor = max(sum(loads) / world, int(counts.max() + np.sort(counts)[:per - 1].sum()))
        assert max(loads) <= 1.05 * floor
        assert balanced_placement(counts, world) == place          # deterministic
    with pytest.raises(ValueError):
        balanced_placement(counts, 5)
