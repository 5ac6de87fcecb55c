/*
 * Which plan a workspace buffer holds.  A plan lives in the caller's buffer, and
 * the matrix descriptor only remembers "my plan is in buffer P".  Two descriptors
 * that are handed the same buffer would each believe that: A1 preprocesses into
 * P, A2 preprocesses into P, and A1's next product would run over A2's tiles.
 * So every plan build takes a fresh serial number, writes it next to the
 * descriptor's record and publishes (buffer -> serial) here; a product reuses
 * the plan in a buffer only while the buffer's published serial is still its
 * own.  The reference keeps such a registry for SpMM, keyed by the workspace
 * address (sparse/spmm/arch35/host/spmm_host.cpp:99-228, an LRU of 1024
 * entries, sparse/spmm/arch35/host/spmm_host_internal.h:56-112); its SpMV
 * records a plan only in Preprocess (sparse/spmv/arch35/spmv_host.cpp:578).
 */
#include <atomic>
#include <cstdint>
#include <list>
#include <mutex>
#include <unordered_map>

#include "aclsparse_b200_kernels.h"
#include "internal.h"
#include "plan_kernels.h"

namespace {

constexpr size_t kMaxEntries = 1024;  // as many as the reference's registry keeps

struct Registry {
    std::mutex mutex;
    std::list<const void*> order;  // most recently published first
    struct Entry {
        uint64_t serial;
        std::list<const void*>::iterator where;
    };
    std::unordered_map<const void*, Entry> entries;
};

Registry& TheRegistry()
{
    static Registry* r = new Registry();  // never destroyed: descriptors may outlive static destructors
    return *r;
}

std::atomic<uint64_t> gNextSerial{1};

}  // namespace

uint64_t AclspPublishPlan(const void* buffer)
{
    const uint64_t serial = gNextSerial.fetch_add(1, std::memory_order_relaxed);
    if (buffer == nullptr) {
        return serial;
    }
    Registry& r = TheRegistry();
    std::lock_guard<std::mutex> lock(r.mutex);
    auto it = r.entries.find(buffer);
    if (it != r.entries.end()) {
        r.order.erase(it->second.where);
        r.entries.erase(it);
    }
    r.order.push_front(buffer);
    r.entries.emplace(buffer, Registry::Entry{serial, r.order.begin()});
    while (r.entries.size() > kMaxEntries) {  // the oldest buffer is forgotten: its plan will be rebuilt
        r.entries.erase(r.order.back());
        r.order.pop_back();
    }
    return serial;
}

bool AclspPlanIsCurrent(const void* buffer, uint64_t serial)
{
    if (buffer == nullptr || serial == 0) {
        return false;
    }
    Registry& r = TheRegistry();
    std::lock_guard<std::mutex> lock(r.mutex);
    const auto it = r.entries.find(buffer);
    return it != r.entries.end() && it->second.serial == serial;
}

namespace {
std::atomic<uint64_t> gLaunches{0};
}

void AclspCountLaunches(unsigned n)
{
    gLaunches.fetch_add(n, std::memory_order_relaxed);
}

extern "C" uint64_t aclsp_b200_kernel_launches(void)
{
    return gLaunches.load(std::memory_order_relaxed);
}
