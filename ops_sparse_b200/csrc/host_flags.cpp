/*
 * Small values that travel from the device to the host without a synchronisation.
 *
 * The SpMV preprocessing pass learns the longest row of the matrix on the device, and the host
 * wants it to pick the kernel for later products, but neither Preprocess nor the product may
 * wait for the device (the reference's arch35 SpMV never synchronises either,
 * sparse/spmv/arch35/spmv_host.cpp:585-632).  So Preprocess enqueues a 4-byte copy from the plan
 * header into a slot of pinned host memory, and a later product simply looks whether the value
 * has arrived; until it has, the product launches both kernels and they decide on the device.
 *
 * Slots come from one pinned block that is allocated on first use and never freed (copies in
 * flight may land after the descriptor that asked for them is gone).  They are handed out round
 * robin; a slot that has been handed out again no longer answers for its earlier holder (the
 * generation check below), which then counts as "not arrived".
 */
#include <atomic>
#include <cstdint>
#include <mutex>

#include <cuda_runtime.h>

#include "internal.h"

namespace {

constexpr uint32_t kSlots = 1u << 16;
constexpr uint32_t kUnknown = 0xFFFFFFFFu;

std::mutex gMutex;
uint32_t* gBlock = nullptr;       // kSlots pinned words
uint64_t* gGeneration = nullptr;  // how often each slot has been handed out
uint32_t gNext = 0;
bool gFailed = false;

}  // namespace

AclspHostSlot AclspAcquireHostSlot()
{
    AclspHostSlot slot;
    std::lock_guard<std::mutex> lock(gMutex);
    if (gBlock == nullptr && !gFailed) {
        void* mem = nullptr;
        if (cudaHostAlloc(&mem, sizeof(uint32_t) * kSlots, cudaHostAllocPortable) != cudaSuccess) {
            (void)cudaGetLastError();
            gFailed = true;  // no pinned memory: values never "arrive", both kernels are launched
        } else {
            gBlock = static_cast<uint32_t*>(mem);
            gGeneration = new uint64_t[kSlots]();
        }
    }
    if (gBlock == nullptr) {
        return slot;
    }
    const uint32_t index = gNext;
    gNext = (gNext + 1u) % kSlots;
    gGeneration[index] += 1;
    reinterpret_cast<volatile uint32_t*>(gBlock)[index] = kUnknown;
    slot.word = gBlock + index;
    slot.index = index;
    slot.generation = gGeneration[index];
    return slot;
}

bool AclspHostSlotValue(const AclspHostSlot& slot, uint32_t* value)
{
    if (slot.word == nullptr) {
        return false;
    }
    {
        std::lock_guard<std::mutex> lock(gMutex);
        if (gGeneration == nullptr || gGeneration[slot.index] != slot.generation) {
            return false;
        }
    }
    const uint32_t v = *reinterpret_cast<const volatile uint32_t*>(slot.word);
    if (v == kUnknown) {
        return false;
    }
    *value = v;
    return true;
}
