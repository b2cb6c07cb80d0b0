// Bounded device-side waits and their host-visible outcome.
//
// Every wait of this library on something another agent produces -- an mbarrier that a TMA
// load or a tcgen05.commit completes, a flag that another GPU writes -- gives up after a
// limit of SM clocks, records a code in the per-device error word and lets the kernel
// leave through its normal teardown, so that a lost producer shows up as an error status
// on the host instead of a hung GPU. This file holds
//   * the cross-rank barrier of the expert-parallel layer (signal pads in peer-mapped
//     memory, plain stores and loads over NVLink, bounded spin),
//   * qs3_moe_check_device_error: error word -> QSFI_STATUS_BACKEND_ERROR,
//   * qs3_debug_bounded_wait_probe: a one-CTA kernel that waits on an mbarrier nobody
//     completes, with a caller-chosen short limit, for testing the expiry path without
//     faulting, trapping or hanging anything.
#include "tcgen05.cuh"

namespace qs3 {

namespace {

enum : uint32_t {
    ERR_EP_BARRIER_WAIT = 0x55000001u,
    ERR_PROBE_WAIT = 0x56000001u,
};

// One block, one thread per peer. Thread q tells rank q "rank `rank` has reached epoch e" by
// storing e into slot `rank` of q's pad, then waits until slot q of its own pad holds an epoch
// >= e (rank q said the same). Epochs only grow, so a fast rank that is already one barrier
// ahead does not confuse a slow one. The stores are release / the loads acquire at system
// scope: what this rank's earlier kernels wrote is visible to a peer that has seen the flag.
__global__ void ep_barrier_kernel(EpBarrierParams p)
{
    const uint32_t q = threadIdx.x;
    // the epoch of this barrier: the caller's, or one more than the device-resident counter (every thread
    // reads it before thread 0, the only writer, can have stored the new value)
    uint32_t epoch = p.epoch;
    if (p.epoch_counter != nullptr)
        epoch = *reinterpret_cast<volatile uint32_t*>(p.epoch_counter) + 1u;
    __syncwarp();
    if (q == 0 && p.epoch_counter != nullptr)
        *reinterpret_cast<volatile uint32_t*>(p.epoch_counter) = epoch;
    if (q >= p.num_ranks)
        return;
    __threadfence_system();
    uint32_t* remote = p.pads[q] + p.my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const uint32_t* mine = p.pads[p.my_rank] + q;
    const uint64_t start = clock64();
    uint32_t spins = 0;
    while (true) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (static_cast<int32_t>(seen - epoch) >= 0)
            return;
        if ((++spins & 15u) != 0)
            continue;
        if (static_cast<uint64_t>(clock64()) - start > p.limit_cycles) {
            if (p.err != nullptr)
                atomicCAS(p.err, 0u, static_cast<uint32_t>(ERR_EP_BARRIER_WAIT));
            return;
        }
    }
}

__global__ void bounded_wait_probe_kernel(uint64_t limit_cycles, uint32_t* err)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // nobody ever arrives on `bar`: the first warp's wait must run into its limit and return;
    // the second warp then sees the raised abort flag in its own wait and returns as well
    if (threadIdx.x == 0)
        tc::mbar_wait<true>(&bar, 0, &abort_flag, err, ERR_PROBE_WAIT, limit_cycles);
    else if (threadIdx.x == 32)
        tc::mbar_wait<false>(&bar, 0, &abort_flag, nullptr, 0, 64 * limit_cycles);
    __syncthreads();
}

} // namespace

cudaError_t launch_ep_barrier(const EpBarrierParams& p, cudaStream_t stream)
{
    ep_barrier_kernel<<<1, 32, 0, stream>>>(p);
    note_launch();
    return cudaGetLastError();
}

} // namespace qs3

using namespace qs3;

extern "C" qsfi_status qs3_moe_ep_barrier(qsfi_context* ctx, const qs3_moe_ep_barrier_desc* d)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (d == nullptr || d->pads == nullptr)
        return set_invalid_arg(ctx, "desc/pads is null");
    if (d->num_ranks == 0 || d->num_ranks > 32 || d->my_rank >= d->num_ranks)
        return set_invalid_arg(ctx, "expert-parallel barrier: 1..32 ranks, my_rank below num_ranks");
    EpBarrierParams p {};
    for (uint32_t r = 0; r < d->num_ranks; ++r) {
        if (d->pads[r] == nullptr || (reinterpret_cast<uintptr_t>(d->pads[r]) & 3u) != 0)
            return set_invalid_arg(ctx, "expert-parallel barrier: pads must be non-null and 4-byte aligned");
        p.pads[r] = static_cast<uint32_t*>(d->pads[r]);
    }
    p.num_ranks = d->num_ranks;
    p.my_rank = d->my_rank;
    p.epoch = d->epoch;
    if (d->epoch_counter != nullptr && (reinterpret_cast<uintptr_t>(d->epoch_counter) & 3u) != 0)
        return set_invalid_arg(ctx, "expert-parallel barrier: epoch_counter must be 4-byte aligned");
    p.epoch_counter = static_cast<uint32_t*>(d->epoch_counter);
    p.limit_cycles = d->timeout_cycles != 0 ? d->timeout_cycles : 4000000000ull; // ~2 s of SM clocks
    p.err = device_error_word();
    return set_cuda_error(ctx, launch_ep_barrier(p, ctx->stream), "qs3_moe_ep_barrier");
}

extern "C" qsfi_status qs3_moe_check_device_error(qsfi_context* ctx)
{
    uint32_t code = 0;
    qsfi_status status = qs3_moe_read_device_error(ctx, &code);
    if (status != QSFI_STATUS_OK)
        return status;
    if (code != 0)
        return set_error(ctx, QSFI_STATUS_BACKEND_ERROR, QSFI_ERROR_SOURCE_QSFI, static_cast<int32_t>(code),
                         "a bounded device-side wait expired (code 0x%08x): a load, a tensor-core commit or a peer "
                         "rank did not arrive in time; results of the affected call are undefined",
                         code);
    return QSFI_STATUS_OK;
}

extern "C" qsfi_status qs3_debug_bounded_wait_probe(qsfi_context* ctx, uint64_t limit_cycles)
{
    if (ctx == nullptr)
        return QSFI_STATUS_INVALID_ARGUMENT;
    clear_error(&ctx->last_error);
    qsfi_status status = activate_context(ctx);
    if (status != QSFI_STATUS_OK)
        return status;
    if (limit_cycles == 0 || limit_cycles > 20000000ull)
        return set_invalid_arg(ctx, "bounded-wait probe: limit of 1 .. 2e7 SM clocks (about 10 ms)");
    bounded_wait_probe_kernel<<<1, 64, 0, ctx->stream>>>(limit_cycles, device_error_word());
    note_launch();
    return set_cuda_error(ctx, cudaGetLastError(), "qs3_debug_bounded_wait_probe");
}
