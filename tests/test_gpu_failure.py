"""Failure detection on the GPU without a GPU fault: every wait of the library's kernels on
something another agent produces is bounded, and an expiry must come back to the host as
``QSFI_STATUS_BACKEND_ERROR`` with the context still usable. The failures here are made by
leaving a producer out (an mbarrier nothing completes, a signal pad nobody writes) and giving
the wait a limit of a fraction of a millisecond; nothing faults, traps or hangs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from qs3_b200 import ops as m
    return m


def _still_usable(ops, ctx):
    logits = torch.tensor([[0.1, 2.0, 2.0, -1.0, 3.0, 0.5]], dtype=torch.float32, device="cuda")
    ids = torch.empty((1, 2), dtype=torch.int32, device="cuda")
    wts = torch.empty((1, 2), dtype=torch.float32, device="cuda")
    ops.router_topk(logits, ids, wts)
    torch.cuda.synchronize()
    assert ids.cpu().tolist() == [[4, 1]]


def test_expired_mbarrier_wait_becomes_a_backend_error(ops):
    """The path every tensor-core kernel takes when a TMA load or a tcgen05.commit never arrives:
    the wait runs into its limit, the kernel returns, the error word holds the code."""
    ctx = ops.Context()
    ctx.check_device_error()                      # nothing pending
    ops.bounded_wait_probe(ctx, 200_000)          # ~0.1 ms of SM clocks
    with pytest.raises(ops.Qs3Error) as e:
        ctx.check_device_error()
    assert e.value.status == ops.capi.STATUS_BACKEND_ERROR
    assert "bounded device-side wait expired" in e.value.message and "0x56000001" in e.value.message
    ctx.check_device_error()                      # reading the word cleared it
    _still_usable(ops, ctx)
    # the raw code is also available to callers that poll instead
    ops.bounded_wait_probe(ctx, 50_000)
    assert ctx.read_device_error() == 0x56000001
    assert ctx.read_device_error() == 0


def test_rank_barrier_times_out_when_a_peer_never_signals(ops):
    """Two "ranks" whose signal pads both live on this GPU. Rank 0 runs the barrier kernel; nothing
    plays rank 1, so slot 1 of rank 0's pad never reaches the epoch and the bounded spin gives up.
    With the slot written beforehand (the peer arrived first) the same call passes."""
    ctx = ops.Context()
    pads = torch.zeros((2, 64), dtype=torch.int32, device="cuda")
    ptrs = [pads[0].data_ptr(), pads[1].data_ptr()]
    ops.ep_barrier(ctx, ptrs, my_rank=0, epoch=1, timeout_cycles=300_000)
    with pytest.raises(ops.Qs3Error) as e:
        ctx.check_device_error()
    assert e.value.status == ops.capi.STATUS_BACKEND_ERROR and "0x55000001" in e.value.message
    got = pads.cpu().numpy()
    assert got[0, 0] == 1 and got[1, 0] == 1       # rank 0 announced itself to both pads before waiting
    assert got[0, 1] == 0
    # the peer is already at epoch 2 (a fast rank one barrier ahead): epochs 2 passes at once
    pads[0, 1] = 2
    ops.ep_barrier(ctx, ptrs, my_rank=0, epoch=2, timeout_cycles=300_000)
    ctx.check_device_error()
    assert pads.cpu().numpy()[1, 0] == 2
    # a single rank is its own peer
    solo = torch.zeros(64, dtype=torch.int32, device="cuda")
    ops.ep_barrier(ctx, [solo.data_ptr()], my_rank=0, epoch=7, timeout_cycles=300_000)
    ctx.check_device_error()
    _still_usable(ops, ctx)
    with pytest.raises(ops.Qs3Error):
        ops.ep_barrier(ctx, ptrs, my_rank=2, epoch=1)


def test_rank_barrier_counts_its_epochs_on_the_device(ops):
    """With an epoch counter in device memory the launch has no per-step argument (that is what lets a
    rank's step be replayed from a CUDA graph): every launch signals counter + 1 and stores it back."""
    ctx = ops.Context()
    solo = torch.zeros(64, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):
        ops.ep_barrier(ctx, [solo.data_ptr()], my_rank=0, epoch=0, timeout_cycles=300_000, epoch_counter=counter)
    ctx.check_device_error()
    assert int(counter.item()) == 3 and int(solo[0].item()) == 3
    # replayed from a graph: three more epochs, nothing expires
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx.use_current_stream()
        with torch.cuda.graph(graph, stream=stream):
            ops.ep_barrier(ctx, [solo.data_ptr()], my_rank=0, epoch=0, timeout_cycles=300_000, epoch_counter=counter)
        for _ in range(3):
            graph.replay()
        stream.synchronize()
    ctx.use_current_stream()
    ctx.check_device_error()
    assert int(counter.item()) == 6 and int(solo[0].item()) == 6
    # a peer that never signals still ends in an error code, not a hang
    pads = torch.zeros((2, 64), dtype=torch.int32, device="cuda")
    ops.ep_barrier(ctx, [pads[0].data_ptr(), pads[1].data_ptr()], my_rank=0, epoch=0, timeout_cycles=300_000,
                   epoch_counter=counter)
    with pytest.raises(ops.Qs3Error) as e:
        ctx.check_device_error()
    assert "0x55000001" in e.value.message
    _still_usable(ops, ctx)


def test_operand_stream_probe_reports_a_plausible_rate(ops):
    """The L2 -> shared-memory probe behind the operand-delivery figures: both tile patterns run to the
    end (no bounded wait expires) and report terabytes per second on an L2-resident buffer."""
    ctx = ops.Context()
    buf = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    for boxes in (False, True):
        gbs = ops.operand_stream_probe(ctx, buf, 16384, 4, 500, boxes=boxes)
        assert 1000.0 < gbs < 40000.0, gbs
    ctx.check_device_error()
    with pytest.raises(ops.Qs3Error):
        ops.operand_stream_probe(ctx, buf, 1000, 4, 10)
