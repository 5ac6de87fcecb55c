/*
 * The node barrier as device code: the stand-alone kernel of gather_kernels.cu and the closing barrier
 * that the last kernel of a sharded product runs in its last CTA (AclspBarrierLink) are the same protocol.
 *
 * A rank announces its next epoch in its slot of every peer's AclspNodeBarrierState (st.release.sys after
 * a system fence, so that what it stored into the peers' buffers before is visible first) and then polls
 * its own slots (ld.acquire.sys) until every peer has announced the epoch too, at most spinLimit polls
 * per peer; a wait that runs out sets the status word and returns.  No trap, no unbounded spin.
 */
#ifndef ACLSPARSE_B200_NODE_BARRIER_CUH_
#define ACLSPARSE_B200_NODE_BARRIER_CUH_

#include <cstdint>

#include "aclsparse_b200_kernels.h"

namespace aclsp {

__device__ __forceinline__ void StoreReleaseSys(uint32_t* addr, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t LoadAcquireSys(const uint32_t* addr)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(addr) : "memory");
    return v;
}

// One warp (all 32 lanes call it); lane r talks to rank r.  peers[r]: rank r's state as this device
// addresses it (entry `rank` unused).
__device__ __forceinline__ void NodeBarrierWarp(AclspNodeBarrierState* local, void* const* peers, uint32_t world,
                                                uint32_t rank, uint32_t spinLimit)
{
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t epoch = 0;
    if (lane == 0) {
        epoch = local->epoch + 1u;
        local->epoch = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    __threadfence_system();  // the stores made before, to any GPU, come first
    const bool peer = lane < world && lane != rank;
    if (peer) {
        StoreReleaseSys(&static_cast<AclspNodeBarrierState*>(peers[lane])->flag[rank], epoch);
    }
    bool arrived = !peer;
    for (uint32_t spin = 0; spin < spinLimit && !arrived; ++spin) {
        // Epochs only grow; the difference is compared so that a wrapped counter still orders.
        arrived = static_cast<int32_t>(LoadAcquireSys(&local->flag[lane]) - epoch) >= 0;
        if (!arrived) {
            __nanosleep(64);
        }
    }
    if (!arrived) {
        atomicExch(&local->status, 1u + lane);  // which peer was missing (the last one to report wins)
    }
}

// Called by EVERY thread of EVERY CTA of the last kernel of a product, after its last store (no thread may
// have returned before).  Each thread fences its stores (plain, peer and multimem stores alike), the CTA
// takes a ticket, and the CTA that draws the last ticket runs the barrier in its first warp.  The ticket
// counter (reserved[0] of the local state) is back at zero when the kernel ends.
__device__ __forceinline__ void CloseWithNodeBarrier(const AclspBarrierLink& link)
{
    if (link.world <= 1u) {
        return;
    }
    __shared__ uint32_t sLastCta;
    auto* local = static_cast<AclspNodeBarrierState*>(link.local);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t ticket = atomicAdd(&local->reserved[0], 1u);
        sLastCta = ticket == gridDim.x * gridDim.y * gridDim.z - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (sLastCta == 0u || threadIdx.x >= 32u) {
        return;
    }
    if (threadIdx.x == 0) {
        local->reserved[0] = 0u;
    }
    __threadfence();  // the tickets of the other CTAs (and the stores they fenced before) are observed
    NodeBarrierWarp(local, link.peers, link.world, link.rank, link.spinLimit);
}

}  // namespace aclsp

#endif  // ACLSPARSE_B200_NODE_BARRIER_CUH_
