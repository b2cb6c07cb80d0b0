"""Expert-parallel MoE layer: one process per GPU, experts split in contiguous blocks,
tokens data-parallel, router and shared expert replicated.

Per layer and rank (T tokens per rank, n ranks):

  1. route     router-logits GEMM + top-k on the rank's own tokens; tokens quantised to
               NVFP4 once (1152 B per row instead of 4096 B of bf16)
  2. dispatch  "pull" (default): the route outputs live in a peer-mapped block; after a barrier over the
               ranks' signal pads every rank copies, with plain peer loads, the ids and weights of all
               tokens and the codes and scales of the tokens that have a route to one of ITS expert
               slots (qs3_moe_ep_pull_routed: a de-duplicated all-to-all, one row per (token, rank)
               pair, no host-side count exchange). With replicated hot experts (below) a token
               reaches ~2.5 of 8 ranks instead of ~7. "gather": all blocks whole
               (qs3_moe_ep_pull_tokens). "nccl": one coalesced group of all-gathers.
  3. experts   the rank's experts over all n*T tokens; routes to other ranks' experts are
               skipped (local_expert_offset), so row t holds the rank's partial sum
  4. combine   "pull": after a second barrier, the owner of a token reads
               the partial sums straight out of the other ranks' buffers (symmetric memory,
               plain peer loads over NVLink) and only for ranks the token has a route to;
               "nccl": all-to-all of the partial sums back to the token owners
  5. finish    shared expert (on a side stream while the dispatch runs) + sum of the n partials in
               ascending rank order in f32 + sigmoid-gated shared term, one bf16 rounding

The barriers between the phases are the library's own (``qs3_moe_ep_barrier``: signal pads in the
peer-mapped block, bounded spin, an expiry is reported by ``check()``); NCCL collectives through
``torch.distributed`` on a separate communication stream when peer mapping is unavailable.
The compute steps are behind a small backend interface so that the exchange logic can
be exercised on CPU ranks (gloo) with a stand-in backend supplied by the tests.
"""
from __future__ import annotations

import statistics

import torch
import torch.distributed as dist

from . import capi, ops


def expert_block(rank: int, world: int, num_experts: int):
    """Contiguous block of experts owned by ``rank``: (first, count)."""
    if num_experts % world != 0:
        raise ValueError("num_experts must be divisible by the number of ranks")
    per = num_experts // world
    return rank * per, per


def balanced_placement(counts, world: int):
    """Static expert placement from routing statistics: a permutation ``placement`` of the
    expert ids such that rank r owns ``placement[r*per:(r+1)*per]`` (``per`` experts each)
    and the per-rank sums of ``counts`` (routes seen per expert on a calibration batch) are
    as even as the longest-processing-time rule makes them: experts in descending count go
    to the least-loaded rank that still has a free slot. Ties keep ascending expert id, so
    every rank computes the same placement from the same counts."""
    counts = [int(c) for c in counts]
    n = len(counts)
    if n % world != 0:
        raise ValueError("num_experts must be divisible by the number of ranks")
    per = n // world
    order = sorted(range(n), key=lambda e: (-counts[e], e))
    loads = [0] * world
    slots = [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(slots[r]) < per), key=lambda r: (loads[r], r))
        slots[r].append(e)
        loads[r] += counts[e]
    return [e for r in range(world) for e in sorted(slots[r])]


def hottest_experts(counts, hot: int):
    """The ``hot`` experts with the most routes (descending count, ties by ascending id)."""
    return sorted(range(len(counts)), key=lambda e: (-int(counts[e]), e))[:hot]


def slot_id_table(num_experts: int, world: int, hot_positions, rank: int):
    """Expert id -> expert SLOT for the tokens that live on ``rank`` when every rank holds, after its
    own ``num_experts / world`` experts, a replica of each expert in ``hot_positions``: slot =
    holder * slots_per_rank + index on the holder; an ordinary expert is held by its owner, a hot
    one by ``rank`` itself (its replica), so routes to hot experts never leave the rank."""
    per = num_experts // world
    slots = per + len(hot_positions)
    hot = {int(p): j for j, p in enumerate(hot_positions)}
    return [rank * slots + per + hot[p] if p in hot else (p // per) * slots + p % per
            for p in range(num_experts)]


class CudaBackend:
    """The three compute phases on this rank's GPU through the C ABI.

    With replicated hot experts (``data.hot_positions``) the plan counts expert SLOTS: every rank
    has ``experts / world`` slots for its own experts plus one per hot expert, and the router's
    ids are mapped to slots (``dispatch_ids``) before the exchange; ``ids`` keeps the router's ids."""

    def __init__(self, ctx: ops.Context, data, world: int):
        import ctypes as C
        self.C = C
        self.ctx, self.data, self.world = ctx, data, world
        cfg = data.cfg
        self.cfg = cfg
        dev = data.hidden.device
        t, h, k, e = cfg.tokens, cfg.hidden, cfg.top_k, cfg.experts
        first, count = data.expert_range
        self.rank = first // count if count else 0
        slots = count + len(getattr(data, "hot_positions", []) or [])
        self.slot_range = (self.rank * slots, slots) if slots != count else (first, count)
        self.id_map = data.slot_id_map(self.rank, world) if slots != count else None
        self.plan = ops.MoePlan(ctx, ops.MoePlanConfig(
            max_num_tokens=t * world, hidden_size=h, intermediate_size=cfg.inter,
            num_experts=e if self.id_map is None else world * slots, top_k=k,
            local_expert_offset=self.slot_range[0], local_num_experts=self.slot_range[1],
            backend=capi.MOE_BACKEND_NVFP4))
        u8, i32, f32, bf = torch.uint8, torch.int32, torch.float32, torch.bfloat16
        self.logits = torch.empty((t, e), dtype=f32, device=dev)
        self.ids = torch.empty((t, k), dtype=i32, device=dev)
        self.dispatch_ids = self.ids if self.id_map is None else torch.empty((t, k), dtype=i32, device=dev)
        self.wts = torch.empty((t, k), dtype=f32, device=dev)
        self.mask = None                 # rank mask per token, bound by the layer when it dispatches by pulling
        self.packed = torch.empty((t, h // 2), dtype=u8, device=dev)
        self.scale = torch.empty((t, h // 16), dtype=u8, device=dev)
        self.ws_experts = torch.empty(self.plan.workspace_size(t * world), dtype=u8, device=dev)
        n = C.c_size_t(0)
        ctx.check(ctx._lib.qs3_moe_ep_finish_workspace_size(ctx.handle, self.plan.handle, t, world,
                                                            cfg.shared_inter, C.byref(n)))
        self.ws_finish = torch.empty(n.value, dtype=u8, device=dev)

    def bind_route_outputs(self, packed, scale, ids, wts, mask=None):
        """Let ``route`` write what the other ranks read into caller-owned tensors (a peer-mapped block)."""
        self.packed, self.scale, self.dispatch_ids, self.wts, self.mask = packed, scale, ids, wts, mask
        if self.id_map is None:
            self.ids = ids

    def pull_routed(self, peer_blocks, offsets, dsts):
        """De-duplicated dispatch: ids / weights of every token, codes / scales of the tokens routed here.
        ``offsets`` = byte offsets of (codes, scales, ids, weights, mask) in a peer block."""
        d = capi.MoeEpPullRoutedDesc()
        self._peer_blocks = (self.C.c_void_p * len(peer_blocks))(*peer_blocks)
        d.peer_blocks = self._peer_blocks
        d.offset_codes, d.offset_scales, d.offset_ids, d.offset_weights, d.offset_mask = offsets
        d.dst_codes, d.dst_scales, d.dst_ids, d.dst_weights = (x.data_ptr() for x in dsts)
        d.num_ranks, d.my_rank = len(peer_blocks), self.rank
        d.num_tokens, d.top_k, d.hidden_size = self.cfg.tokens, self.cfg.top_k, self.cfg.hidden
        self.ctx.check(self.ctx._lib.qs3_moe_ep_pull_routed(self.ctx.handle, self.C.byref(d)))

    def pull_tokens(self, peer_blocks, offsets, sizes, dsts):
        """All-gather by peer loads: segment j of every rank's block -> dsts[j][rank]."""
        d = capi.MoeEpPullTokensDesc()
        self._peer_blocks = (self.C.c_void_p * len(peer_blocks))(*peer_blocks)
        d.peer_blocks = self._peer_blocks
        for j, (off, size, dst) in enumerate(zip(offsets, sizes, dsts)):
            d.segment_offset[j], d.segment_bytes[j], d.dst[j] = off, size, dst.data_ptr()
        d.num_ranks, d.num_segments = len(peer_blocks), len(offsets)
        self.ctx.check(self.ctx._lib.qs3_moe_ep_pull_tokens(self.ctx.handle, self.C.byref(d)))

    def route(self, hidden):
        d = capi.MoeEpRouteDesc()
        dt = self.data
        d.hidden = ops._desc(hidden, 2)
        d.router_weight = ops._desc(dt.router, 2)
        d.router_bias = ops._desc(dt.bias, 1)
        d.router_logits = ops._desc(self.logits, 2)
        d.topk_ids = ops._desc(self.ids, 2)
        d.topk_weights = ops._desc(self.wts, 2)
        d.hidden_packed = ops._desc(self.packed, 2)
        d.hidden_scale = ops._desc(self.scale, 2, capi.DTYPE_FP8_E4M3)
        d.score, d.renormalize, d.routed_scaling_factor, d.act_global_scale = 0, 1, 1.0, 1.0
        d.num_tokens = hidden.shape[0]
        if self.id_map is not None:
            d.expert_id_map = ops._desc(self.id_map, 1)
            d.dispatch_ids = ops._desc(self.dispatch_ids, 2)
        if self.mask is not None:
            d.rank_mask = ops._desc(self.mask, 1)
            d.num_ranks = self.world
        self.ctx.check(self.ctx._lib.qs3_moe_ep_route(self.ctx.handle, self.plan.handle, self.C.byref(d)))
        return self.packed, self.scale, self.dispatch_ids, self.wts

    def experts(self, packed, scale, ids, wts, out, skip_empty=False):
        d = capi.MoeNvfp4PreparedDesc()
        dt = self.data
        d.hidden_packed = ops._desc(packed, 2)
        d.hidden_scale = ops._desc(scale, 2, capi.DTYPE_FP8_E4M3)
        d.topk_ids = ops._desc(ids, 2)
        d.topk_weights = ops._desc(wts, 2)
        d.gate_up_weight = ops._desc(dt.gate_up.packed, 3)
        d.gate_up_scale_tiled = ops._desc(dt.gate_up.scale_tiled, 1)
        d.gate_up_global_scale = ops._desc(dt.gate_up.global_scale, 1)
        d.down_weight = ops._desc(dt.down.packed, 3)
        d.down_scale_tiled = ops._desc(dt.down.scale_tiled, 1)
        d.down_global_scale = ops._desc(dt.down.global_scale, 1)
        d.act_global_scale = d.act2_global_scale = 1.0
        d.out = ops._desc(out, 2)
        d.workspace = ops._desc(self.ws_experts, 1)
        d.num_tokens = packed.shape[0]
        d.flags = 1 if skip_empty else 0
        self.ctx.check(self.ctx._lib.qs3_moe_execute_nvfp4_prepared(self.ctx.handle, self.plan.handle,
                                                                    self.C.byref(d)))

    def _finish(self, hidden, partials, out, phases, peer_ptrs=None, ids=None):
        d = capi.MoeEpFinishDesc()
        if peer_ptrs is not None:
            self._peer_array = (self.C.c_void_p * len(peer_ptrs))(*peer_ptrs)
            d.peer_partials = self._peer_array
            d.topk_ids = ops._desc(ids, 2)
        sh = self.data.shared
        d.hidden = ops._desc(hidden, 2)
        d.partials = ops._desc(partials, 3)
        if sh is not None:
            d.shared_gate_up_weight = ops._desc(sh.gate_up.packed, 3)
            d.shared_gate_up_scale_tiled = ops._desc(sh.gate_up.scale_tiled, 1)
            d.shared_gate_up_global_scale = ops._desc(sh.gate_up.global_scale, 1)
            d.shared_down_weight = ops._desc(sh.down.packed, 3)
            d.shared_down_scale_tiled = ops._desc(sh.down.scale_tiled, 1)
            d.shared_down_global_scale = ops._desc(sh.down.global_scale, 1)
            d.shared_gate_weight = ops._desc(sh.gate_weight, 2)
            d.shared_intermediate_size = sh.intermediate_size
        d.act_global_scale = d.act2_global_scale = 1.0
        d.out = ops._desc(out, 2)
        d.workspace = ops._desc(self.ws_finish, 1)
        d.num_tokens, d.num_ranks, d.phases = hidden.shape[0], self.world, phases
        self.ctx.check(self.ctx._lib.qs3_moe_ep_finish(self.ctx.handle, self.plan.handle, self.C.byref(d)))

    def shared_expert(self, hidden):
        if self.data.shared is not None:
            self._finish(hidden, None, None, 1)

    def finish(self, hidden, partials, out):
        self._finish(hidden, partials, out, 2)

    def finish_pull(self, hidden, peer_ptrs, ids, out):
        """Phase 2 reading every rank's partial sums in place (peer-mapped pointers)."""
        self._finish(hidden, None, out, 2, peer_ptrs=peer_ptrs, ids=ids)


class ExpertParallelLayer:
    """Drives one layer across the ranks of the default process group."""

    def __init__(self, ctx, data, rank: int, world: int, backend=None, group=None, combine="auto",
                 dispatch="auto"):
        self.rank, self.world, self.group = rank, world, group
        self.barrier_timeout_cycles = 0          # library default (about two seconds of SM clocks)
        self.graph = None                        # CUDA graph of one resident-input step (capture())
        self.launches_per_step = 0
        self.data = data
        cfg = data.cfg
        self.cfg = cfg
        self.backend = backend if backend is not None else CudaBackend(ctx, data, world)
        self.ctx = ctx
        dev = data.hidden.device
        self.cuda = dev.type == "cuda"
        t, h, k = cfg.tokens, cfg.hidden, cfg.top_k
        n = world
        u8, i32, f32, bf = torch.uint8, torch.int32, torch.float32, torch.bfloat16
        # gathered token buffers: rank r's tokens occupy rows [r*T, (r+1)*T)
        self.g_packed = torch.empty((n * t, h // 2), dtype=u8, device=dev)
        self.g_scale = torch.empty((n * t, h // 16), dtype=u8, device=dev)
        self.g_ids = torch.empty((n * t, k), dtype=i32, device=dev)
        self.g_wts = torch.empty((n * t, k), dtype=f32, device=dev)
        # this rank's partial sums for all n*T tokens. On GPUs it lives in symmetric memory so
        # that the owners of the tokens can read it in place over NVLink ("pull" combine);
        # when that cannot be set up the partial sums are exchanged with an NCCL all-to-all.
        self.peer_ptrs = None
        self.partial = None
        self.token_block = None
        if self.cuda and world > 1 and combine != "nccl":
            try:
                import os
                # only plain peer loads and stores touch the block: no NVLink multicast object is wanted
                os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
                import torch.distributed._symmetric_memory as symm
                # one peer-mapped block per rank: [partial sums | codes | scales | ids | weights | signal pads]
                sizes = [n * t * h * 2, t * (h // 2), t * (h // 16), t * k * 4, t * k * 4, 2 * 256, t * 4]
                offs, total = [], 0
                for sz in sizes:
                    offs.append(total)
                    total += (sz + 255) // 256 * 256
                self._sym = symm.empty((total,), dtype=u8, device=dev)
                hdl = symm.rendezvous(self._sym, dist.group.WORLD if group is None else group)
                self._symm_handle = hdl
                base = [int(ptr) for ptr in hdl.buffer_ptrs]
                self.partial = self._sym[offs[0]:offs[0] + sizes[0]].view(bf).view(n * t, h)
                self.peer_ptrs = [b + offs[0] for b in base]
                # signal pads of the library's own bounded barrier: two channels of n words per rank
                self._sym[offs[5]:offs[5] + sizes[5]].zero_()
                torch.cuda.synchronize(dev)
                dist.barrier(group=group)        # every pad is zero before anybody signals
                self._pads = [[b + offs[5] + 256 * ch for b in base] for ch in range(2)]
                # epochs are counted on the device (one word per channel), so a barrier launch has no
                # per-step argument and the whole step can be replayed from a CUDA graph
                self._epoch_dev = torch.zeros(2, dtype=torch.int32, device=dev)
                if dispatch != "nccl" and hasattr(self.backend, "bind_route_outputs"):
                    seg = lambda j, dt, shape: self._sym[offs[j]:offs[j] + sizes[j]].view(dt).view(shape)
                    routed = dispatch != "gather" and h % 256 == 0 and h <= 2048
                    self.backend.bind_route_outputs(seg(1, u8, (t, h // 2)), seg(2, u8, (t, h // 16)),
                                                    seg(3, i32, (t, k)), seg(4, f32, (t, k)),
                                                    seg(6, i32, (t,)) if routed else None)
                    self.token_block = dict(peers=base, offsets=offs[1:5], sizes=sizes[1:5],
                                            routed=offs[1:5] + [offs[6]] if routed else None)
            except Exception as exc:  # no peer mapping on this system: exchange copies instead
                if combine == "pull":
                    raise
                self.partial, self.peer_ptrs, self.combine_note = None, None, f"nccl ({type(exc).__name__})"
                self.token_block = None
        if self.partial is None:
            self.partial = torch.empty((n * t, h), dtype=bf, device=dev)
        self.combine_mode = "pull" if self.peer_ptrs is not None else "nccl"
        self.dispatch_mode = "pull" if self.token_block is not None else "nccl"
        self.flag = torch.zeros(1, dtype=f32, device=dev) if self.cuda else None
        self.recv = torch.empty((n, t, h), dtype=bf, device=dev)        # partial sums of my tokens, per rank
        self.out = torch.empty((t, h), dtype=bf, device=dev)
        self.x_dev = torch.empty((t, h), dtype=bf, device=dev)
        if self.cuda:
            self.comm = torch.cuda.Stream(device=dev)
            self.ev = [torch.cuda.Event() for _ in range(4)]

    # -- collectives (NCCL on the communication stream; gloo in the CPU tests) --
    def _dispatch(self, packed, scale, ids, wts):
        try:
            self._dispatch_collectives(packed, scale, ids, wts)
        except RuntimeError as exc:
            # a rank that died or never joined: the process group's timeout ends the collective
            raise ops.Qs3Error(capi.STATUS_BACKEND_ERROR, f"expert-parallel dispatch failed: {exc}") from exc

    def _dispatch_collectives(self, packed, scale, ids, wts):
        pairs = ((self.g_packed, packed), (self.g_scale, scale), (self.g_ids, ids), (self.g_wts, wts))
        if self.cuda:
            # one NCCL group for the four gathers instead of four launches
            with dist._coalescing_manager(group=self.group, device=packed.device, async_ops=False):
                for dst, src in pairs:
                    dist.all_gather_into_tensor(dst, src, group=self.group)
        else:
            for dst, src in pairs:
                dist.all_gather_into_tensor(dst, src, group=self.group)

    def _barrier(self, channel: int):
        """The library's barrier over the ranks' signal pads, on the current stream. Its wait is
        bounded: a rank that never arrives leaves an error code that ``check()`` raises."""
        ops.ep_barrier(self.ctx, self._pads[channel], self.rank, 0, self.barrier_timeout_cycles,
                       epoch_counter=self._epoch_dev[channel:channel + 1])

    def check(self):
        """Synchronise and raise if a bounded device-side wait of the steps so far expired."""
        if self.cuda and self.ctx is not None:
            self.ctx.check_device_error()

    def _dispatch_pull(self):
        """Barrier over the ranks' signal pads (every rank's route outputs are in its block),
        then copy all blocks here with peer loads."""
        tb = self.token_block
        self._barrier(0)
        if tb["routed"] is not None:
            # every token row crosses NVLink once per rank that holds one of its experts
            self.backend.pull_routed(tb["peers"], tb["routed"], (self.g_packed, self.g_scale, self.g_ids, self.g_wts))
        else:
            self.backend.pull_tokens(tb["peers"], tb["offsets"], tb["sizes"],
                                     (self.g_packed, self.g_scale, self.g_ids, self.g_wts))

    def _combine(self):
        try:
            dist.all_to_all_single(self.recv.view(self.world * self.cfg.tokens, -1), self.partial, group=self.group)
        except RuntimeError as exc:
            raise ops.Qs3Error(capi.STATUS_BACKEND_ERROR, f"expert-parallel combine failed: {exc}") from exc

    def capture(self):
        """Record one resident-input step (this rank's share of it: its kernels, the peer loads and the
        two barriers) in a CUDA graph. Eager, a step is about ten library calls of 30-40 us of host time
        each, which is as long as the GPU work of a rank at 4 or 8 GPUs. Every rank must capture, and
        every rank must then replay the same number of steps (the barriers count their epochs on the
        device). Only the peer-load paths are capturable; with NCCL in the step this is a no-op."""
        if not (self.cuda and self.combine_mode == "pull" and self.dispatch_mode == "pull") or self.graph is not None:
            return
        for _ in range(2):
            self.step()
        torch.cuda.synchronize()
        before = ops.launch_count()
        self.step()
        self.launches_per_step = ops.launch_count() - before
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: the process group's watchdog thread keeps querying its own events
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self._step_eager(self.data.hidden, self.out)
        self.ctx.use_current_stream()
        self.graph = graph

    def try_capture(self):
        """``capture`` on every rank; falls back to eager launches on all ranks if any rank failed."""
        ok = 1.0
        try:
            self.capture()
        except Exception as exc:
            import sys
            print(f"rank {self.rank}: CUDA graph capture failed ({exc}); eager launches", file=sys.stderr)
            ok = 0.0
            torch.cuda.synchronize()
        if self.cuda and self.world > 1:
            flag = torch.tensor([ok], device=self.data.hidden.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            ok = float(flag.item())
        if ok == 0.0:
            self.graph = None
            if self.ctx is not None and self.cuda:
                self.ctx.use_current_stream()

    def step(self, hidden=None, out=None):
        if self.graph is not None and hidden is None and out is None:
            self.graph.replay()
            return self.out
        return self._step_eager(self.data.hidden if hidden is None else hidden, self.out if out is None else out)

    def _step_eager(self, hidden, out):
        b = self.backend
        if self.cuda and self.ctx is not None:
            self.ctx.use_current_stream()
        packed, scale, ids, wts = b.route(hidden)
        if not self.cuda:
            self._dispatch(packed, scale, ids, wts)
            b.shared_expert(hidden)
            b.experts(self.g_packed, self.g_scale, self.g_ids, self.g_wts, self.partial)
            self._combine()
            b.finish(hidden, self.recv, out)
            return out
        main = torch.cuda.current_stream()
        pull = self.combine_mode == "pull"
        self.ev[0].record(main)
        if self.dispatch_mode == "pull":
            # shared expert on the side stream while barrier + peer copies run on the main one
            self.comm.wait_event(self.ev[0])
            self.ctx.set_stream(self.comm.cuda_stream)
            b.shared_expert(hidden)
            self.ctx.set_stream(main.cuda_stream)
            self.ev[1].record(self.comm)
            self._dispatch_pull()
        else:
            with torch.cuda.stream(self.comm):
                self.comm.wait_event(self.ev[0])
                self._dispatch(packed, scale, ids, wts)
                self.ev[1].record(self.comm)
            b.shared_expert(hidden)              # overlaps the dispatch
            main.wait_event(self.ev[1])
        b.experts(self.g_packed, self.g_scale, self.g_ids, self.g_wts, self.partial, skip_empty=pull)
        if pull and self.dispatch_mode == "pull":
            # every rank's partial sums are complete once all ranks passed this barrier; the
            # barrier of the next step's dispatch keeps anyone from overwriting a buffer early
            self._barrier(1)
            main.wait_event(self.ev[1])
            b.finish_pull(hidden, self.peer_ptrs, ids, out)
            return out
        self.ev[2].record(main)
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(self.ev[2])
            if pull:
                # a one-element all-reduce as the cross-rank barrier: it completes here only
                # after every rank's stream has passed its experts phase. The next step's
                # dispatch all-gather is the barrier in the other direction (nobody overwrites
                # a partial-sum buffer before all ranks finished reading it).
                dist.all_reduce(self.flag, group=self.group)
            else:
                self._combine()
            self.ev[3].record(self.comm)
        main.wait_event(self.ev[3])
        if pull:
            b.finish_pull(hidden, self.peer_ptrs, ids, out)
        else:
            b.finish(hidden, self.recv, out)
        return out

    def routing_snapshot(self):
        """What the last step's experts phase sorted on this rank, as numpy arrays: (ids, weights)
        of every token row it saw, the rank's expert range, and the plan's routing tables
        (counts, indptr, route_rows, row_tokens). For parity checks."""
        b = self.backend
        first, count = getattr(b, "slot_range", self.data.expert_range)
        tables = b.plan.routing_tables(b.ws_experts, self.g_ids.shape[0])
        return (self.g_ids.cpu().numpy(), self.g_wts.cpu().numpy(), first, count,
                [x.cpu().numpy() for x in tables[:4]])

    # -- measurement helpers used by bench.py --
    def profile(self, iters):
        """Mean ms of the phases, timed with CUDA events on a serialised pass."""
        names = ("route", "dispatch", "shared_expert", "experts", "combine_exchange", "finish")
        acc = {k: [] for k in names}
        b = self.backend
        hidden = self.data.hidden
        for _ in range(iters):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(7)]
            if self.cuda and self.world > 1:
                # ranks start each pass together, so "dispatch" holds the gather itself and
                # "combine_exchange" the wait for the slowest rank's experts phase
                dist.barrier(group=self.group)
                torch.cuda.synchronize()
            ev[0].record()
            packed, scale, ids, wts = b.route(hidden)
            ev[1].record()
            if self.dispatch_mode == "pull":
                self._dispatch_pull()
            else:
                self._dispatch(packed, scale, ids, wts)
            ev[2].record()
            b.shared_expert(hidden)
            ev[3].record()
            pull = self.combine_mode == "pull"
            sub = self.cuda and hasattr(b, "ctx")
            if sub:
                ops.profile_begin(b.ctx)
            b.experts(self.g_packed, self.g_scale, self.g_ids, self.g_wts, self.partial, skip_empty=pull)
            ev[4].record()
            if sub:  # stages inside the experts phase, recorded by the library
                for name, ms in ops.profile_end(b.ctx):
                    acc.setdefault("experts/" + name, []).append(ms)
            if pull and self.dispatch_mode == "pull":
                self._barrier(1)
            elif pull:
                dist.all_reduce(self.flag, group=self.group)
            else:
                self._combine()
            ev[5].record()
            if pull:
                b.finish_pull(hidden, self.peer_ptrs, ids, self.out)
            else:
                b.finish(hidden, self.recv, self.out)
            ev[6].record()
            torch.cuda.synchronize()
            for i, name in enumerate(names):
                acc[name].append(ev[i].elapsed_time(ev[i + 1]))
        return {k: statistics.mean(v) for k, v in acc.items() if v}

    def roofline(self, stage_ms, hbm_gbs, peak_kind):
        """Dominant kernel at n > 1 as at n = 1: the grouped gate_up GEMM + SwiGLU of the local experts,
        timed by the library's stage events inside the experts phase. Algorithmic bytes = gate_up
        weights of this rank's expert slots that received rows + the quantised rows read and written;
        FLOPs = 2 * local routes * 2I * H; the bound is whichever takes longer at its measured peak.
        `nvlink` describes the combine exchange: bytes this rank pulled from its peers (one bf16 partial
        row per (token, remote rank) pair that has a route), the time of the pulling kernel and its
        fraction of a peer copy measured with the library's own copy kernel on a large buffer."""
        cfg = self.cfg
        ms = stage_ms.get("experts/gate_up_gemm_swiglu")
        if not ms:
            return None
        first, count = getattr(self.backend, "slot_range", self.data.expert_range)
        ids = self.g_ids.flatten().long()
        local = ids[(ids >= first) & (ids < first + count)] - first
        counts = torch.bincount(local, minlength=count)
        hit = int((counts > 0).sum().item())
        routes = int(local.numel())
        gu_b, _d_b = self.data.weight_bytes_per_expert()
        row_in, row_out = cfg.hidden // 2 + cfg.hidden // 16, cfg.inter // 2 + cfg.inter // 16
        algo = hit * gu_b + routes * (row_in + row_out)
        flops = 2.0 * routes * 2 * cfg.inter * cfg.hidden
        ceiling = ops.tensor_peak_probe(self.ctx, "nvfp4", 256, 20000)
        t_hbm, t_tensor = algo / (hbm_gbs * 1e9), flops / (ceiling * 1e12)
        tflops, gbs = flops / (ms * 1e-3) / 1e12, algo / (ms * 1e-3) / 1e9
        tensor_bound = t_tensor > t_hbm
        out = {"bound": "tensor" if tensor_bound else "hbm", "achieved": tflops if tensor_bound else gbs,
               "peak": ceiling if tensor_bound else hbm_gbs, "unit": "TFLOP/s" if tensor_bound else "GB/s",
               "frac": tflops / ceiling if tensor_bound else gbs / hbm_gbs, "traffic": None,
               "peak_source": ("measured in this run: issue loop of 128 x 256 tcgen05.mma on resident tiles, every SM"
                               if tensor_bound else f"{peak_kind} copy bandwidth"),
               "kernel": "grouped gate_up GEMM + SwiGLU of the rank's expert slots (rank 0)", "kernel_ms": ms,
               "algorithmic_bytes": algo, "algorithmic_flops": flops, "experts_hit": hit, "local_routes": routes,
               "max_rows_per_expert": int(counts.max().item()) if count else 0,
               "hbm_gbs": gbs, "hbm_frac": gbs / hbm_gbs, "tensor_tflops": tflops,
               "tensor_ceiling_tflops": ceiling, "tensor_frac_of_measured_ceiling": tflops / ceiling,
               "experts_phase_ms": stage_ms.get("experts")}
        finish = stage_ms.get("finish")
        if self.combine_mode == "pull" and finish:
            mine = self.backend.dispatch_ids.long() // count           # rank each route goes to
            remote = 0
            for r in range(self.world):
                if r != self.rank:
                    remote += int((mine == r).any(dim=1).sum().item())
            pulled = remote * cfg.hidden * 2
            peak = self.measure_peer_copy()
            out["nvlink"] = {"bytes_pulled": pulled, "finish_ms": finish,
                             "achieved_gbs": pulled / (finish * 1e-3) / 1e9, "peak_gbs_measured": peak,
                             "frac": (pulled / (finish * 1e-3) / 1e9 / peak) if peak else None,
                             "partial_rows_per_token": remote / cfg.tokens,
                             "note": "finish = pull of the partial sums over NVLink + ordered sum + shared expert "
                                     "gate, one kernel; peak = a 256 MB copy from the next rank's memory with "
                                     "the library's peer-copy kernel"}
        return out

    def measure_peer_copy(self, mbytes: int = 256):
        """GB/s of copying `mbytes` MB out of the next rank's peer-mapped memory with the library's own
        peer-copy kernel (plain 16-byte loads over NVLink), CUDA events, best of three."""
        if not self.cuda or self.world < 2 or self.token_block is None:
            return None
        import torch.distributed._symmetric_memory as symm
        nbytes = mbytes << 20
        dev = self.data.hidden.device
        buf = symm.empty((nbytes,), dtype=torch.uint8, device=dev)
        hdl = symm.rendezvous(buf, dist.group.WORLD if self.group is None else self.group)
        peers = [int(p) for p in hdl.buffer_ptrs]
        src = peers[(self.rank + 1) % self.world]
        dst = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        best = 0.0
        for _ in range(4):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier(group=self.group)
            torch.cuda.synchronize(dev)
            a.record()
            self.backend.pull_tokens([src], [0], [nbytes], (dst,))
            b.record()
            torch.cuda.synchronize(dev)
            best = max(best, nbytes / (a.elapsed_time(b) * 1e-3) / 1e9)
        dist.barrier(group=self.group)
        del dst, buf, hdl
        return best
