/*
 * Reassembly of y / C across the GPUs of one node by peer stores.
 *
 * Each rank owns a contiguous block of rows of the result.  After its product
 * it writes that block into the result buffer of every other rank through
 * peer-mapped pointers (plain 128-bit stores over NVLink / NVSwitch): one
 * launch, all peers at once, no staging copy and no collective library call.
 * Ranks then meet at the node barrier below.  No TMA, no multicast load: every
 * access to a peer's memory here is an ordinary store.
 *
 * Node barrier.  Every rank keeps an AclspNodeBarrierState in peer-mapped
 * memory.  A barrier is one tiny kernel per rank: it counts the rank's epoch
 * up, stores the epoch into its own slot of every peer's flag array
 * (st.release.sys, after a system-wide fence, so that the row blocks stored by
 * the kernels before it are visible first), then polls its own flag array
 * until every peer has announced the same epoch (ld.acquire.sys).  The poll is
 * bounded: when a peer does not show up within the limit the kernel sets the
 * state's status word and returns, the host reads it
 * (aclsparseB200NodeBarrierStatus) and reports ACL_SPARSE_STATUS_EXECUTION_FAILED.
 * Nothing traps and nothing spins without a limit, so a rank that is gone
 * costs its peers the limit, not the GPU.
 *
 * The reference library is single-device; this file has no counterpart there.
 */
#include <cstdint>

#include <cuda_runtime.h>

#include "aclsparse_b200_kernels.h"
#include "node_barrier.cuh"
#include "plan_kernels.h"

namespace {

constexpr int kMaxPeers = 16;

struct PeerList {
    float* ptr[kMaxPeers];
};

// grid.y selects the peer; the block of `count` floats at element `offset` is
// copied from `src` (this rank's buffer) to the same place in the peer's buffer.
__global__ void PushSliceKernel(const float* __restrict__ src, PeerList peers, int64_t offset, int64_t count)
{
    float* __restrict__ dst = peers.ptr[blockIdx.y] + offset;
    const float* __restrict__ from = src + offset;
    // Where both sides sit at the same offset of equally aligned buffers, one prologue brings both
    // to a 16-byte boundary and the body moves 16-byte vectors; a peer buffer aligned differently
    // from the source gets plain 4-byte stores throughout.
    const bool sameAlignment = ((reinterpret_cast<uintptr_t>(from) ^ reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    const int64_t mis = (reinterpret_cast<uintptr_t>(from) & 15u) / 4u;
    int64_t head = mis == 0 ? 0 : 4 - mis;
    head = sameAlignment ? (head < count ? head : count) : count;
    const int64_t vecs = (count - head) / 4;
    const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = tid; i < head; i += step) {
        dst[i] = from[i];
    }
    const float4* from4 = reinterpret_cast<const float4*>(from + head);
    float4* dst4 = reinterpret_cast<float4*>(dst + head);
    for (int64_t v = tid; v < vecs; v += step) {
        dst4[v] = from4[v];
    }
    const int64_t tail = head + 4 * vecs;
    if (tid < count - tail) {
        dst[tail + tid] = from[tail + tid];
    }
}

struct BarrierPeers {
    AclspNodeBarrierState* ptr[ACLSP_BARRIER_MAX_RANKS];
};

// One warp; lane r talks to rank r.
__global__ void NodeBarrierKernel(AclspNodeBarrierState* local, BarrierPeers peers, uint32_t world, uint32_t rank,
                                  uint32_t spinLimit)
{
    aclsp::NodeBarrierWarp(local, reinterpret_cast<void* const*>(peers.ptr), world, rank, spinLimit);
}

}  // namespace

extern "C" void aclsp_b200_node_barrier_kernel_do(void* localState, void* const* peerStates, uint32_t world,
                                                  uint32_t rank, uint32_t spinLimit, void* stream)
{
    if (world <= 1 || world > ACLSP_BARRIER_MAX_RANKS || rank >= world) {
        return;
    }
    BarrierPeers peers{};
    for (uint32_t r = 0; r < world; ++r) {
        peers.ptr[r] = static_cast<AclspNodeBarrierState*>(peerStates[r]);
    }
    AclspCountLaunches(1);
    NodeBarrierKernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<AclspNodeBarrierState*>(localState), peers, world, rank, spinLimit);
}

extern "C" void aclsp_b200_push_slice_kernel_do(const void* src, void* const* peers, uint32_t numPeers,
                                                int64_t offsetElems, int64_t countElems, void* stream)
{
    if (numPeers == 0 || countElems <= 0) {
        return;
    }
    // A launch serves up to kMaxPeers peers; longer lists take further launches.
    for (uint32_t first = 0; first < numPeers; first += kMaxPeers) {
        PeerList list{};
        const uint32_t n = numPeers - first > kMaxPeers ? kMaxPeers : numPeers - first;
        for (uint32_t i = 0; i < n; ++i) {
            list.ptr[i] = static_cast<float*>(peers[first + i]);
        }
        // Enough blocks to keep the links busy, few enough to launch quickly.
        int64_t blocks = (countElems / 4 + 255) / 256;
        blocks = blocks < 1 ? 1
                            : (blocks > 592 / static_cast<int64_t>(n) + 1 ? 592 / static_cast<int64_t>(n) + 1 : blocks);
        const dim3 grid(static_cast<unsigned>(blocks), n);
        AclspCountLaunches(1);
        PushSliceKernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const float*>(src), list,
                                                                            offsetElems, countElems);
    }
}
