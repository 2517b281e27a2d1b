// Barrier between the GPUs of one node (one process per GPU), used after the attention kernel has stored its
// head-sharded output rows straight into every GPU's gathered buffer.
//
// Every rank owns a flag array uint32[RQ_MAX_PEERS] that all ranks have mapped (CUDA IPC): slot r is written only by
// rank r.  A launch takes the next epoch from this rank's device-side counter, publishes it in slot `rank` of every
// rank's array with a system-scope release store, then waits until every slot of its own array has reached the epoch.
// The stores of earlier kernels in the same stream are ordered before the flag by the kernel boundary plus the
// release; the acquire loads plus this kernel's completion order them before whatever the stream runs next.
// The epoch is device state, so a captured launch stays valid across CUDA-graph replays.
//
// The wait is bounded twice (global timer and a poll count).  On expiry the kernel records RQ_ERR_DEVICE_TIMEOUT and
// returns; it never traps and never spins without limit.  Ranks wait for kernels running on OTHER GPUs only: never
// launch two ranks of one barrier on the same GPU.
#include "rq_common.cuh"
#include "rq_kernels.h"

namespace rq {
namespace {

constexpr unsigned long long kMaxPolls = 200ull * 1000 * 1000;

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void store_release_system(uint32_t* address, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(address), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* address) {
    uint32_t value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ PeerBarrierParams p) {
    __shared__ uint32_t next_epoch;
    const int t = threadIdx.x;
    // Launched as a programmatic dependent: the CTA is resident while the kernel in front of it (the attention call whose
    // stores this barrier covers) still runs, and starts the moment that kernel has completed and flushed.  The kernel
    // behind it may be scheduled at once; it waits for this grid's completion itself.
    pdl_wait();
    pdl_launch_dependents();
    if (t == 0) {
        // wait-only: the epoch was advanced and published by this rank's attention kernels; just wait for the peers
        next_epoch = p.wait_only ? p.state[0] : p.state[0] + 1u;
        if (!p.wait_only) p.state[0] = next_epoch;
    }
    __syncwarp();
    const uint32_t epoch = next_epoch;
    if (t >= p.world) return;
    // The release store is itself a system-scope fence followed by the store; what it has to cover -- the rows the
    // previous kernel stored into the peers' buffers -- was completed by that kernel's end, which this kernel waited for.
    if (!p.wait_only) store_release_system(p.flags[t] + p.rank, epoch);
    const uint32_t* arrival = p.flags[p.rank] + t;
    const unsigned long long start = global_timer_ns();
    for (unsigned long long polls = 0;; ++polls) {
        // a fast peer may already be one barrier ahead: compare as a signed distance
        if (static_cast<int32_t>(load_acquire_system(arrival) - epoch) >= 0) return;
        if (polls > 32) __nanosleep(200);
        if (polls > kMaxPolls || global_timer_ns() - start > p.timeout_ns) {
            atomicExch(p.state + 1, static_cast<uint32_t>(RQ_ERR_DEVICE_TIMEOUT));
            return;
        }
    }
}

}  // namespace

cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(1);
    config.blockDim = dim3(32);
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = p.programmatic_launch ? 1 : 0;
    return cudaLaunchKernelEx(&config, peer_barrier_kernel, p);
}

}  // namespace rq
