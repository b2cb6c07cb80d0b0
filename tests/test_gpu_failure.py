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
