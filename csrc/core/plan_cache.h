// Launch-plan cache.
//
// HCCL amortises the host cost of an operator in three places: the AICPU task
// cache (kernel_launch.cc:842-962), the CCU fast launch (op_common.cc:348-466:
// when an op needs one loop, cache the handles and up to 48 task args and skip
// selector + resource path next time) and the AIV instruction cache
// (hccl_aiv_utils.h:189-217: FNV hash of (comm, count, dtype, op, root, blocks,
// engine), 8192-entry ring, 20 % eviction).  Here a plan is the outcome of
// selection for one call signature: device algorithm, block count and chunking;
// a hit skips the cost table and the constraint checks.
#pragma once
#include <cstdint>
#include <algorithm>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace hccl {

struct PlanKey {
    uint32_t op, dtype, redOp, root;
    uint64_t bytes;
    uint32_t flags;      // registration / alignment / in-place bits that selection depends on
    uint32_t generation; // communicator generation (bumped by resume)
    bool operator==(const PlanKey& o) const
    {
        return op == o.op && dtype == o.dtype && redOp == o.redOp && root == o.root && bytes == o.bytes && flags == o.flags &&
               generation == o.generation;
    }
};

inline uint64_t Fnv1a(const void* data, size_t n, uint64_t h = 1469598103934665603ull)
{
    const unsigned char* p = (const unsigned char*)data;
    for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 1099511628211ull; }
    return h;
}
struct PlanKeyHash {
    size_t operator()(const PlanKey& k) const
    {
        uint64_t h = Fnv1a(&k.op, sizeof(k.op));
        h = Fnv1a(&k.dtype, sizeof(k.dtype), h);
        h = Fnv1a(&k.redOp, sizeof(k.redOp), h);
        h = Fnv1a(&k.root, sizeof(k.root), h);
        h = Fnv1a(&k.bytes, sizeof(k.bytes), h);
        h = Fnv1a(&k.flags, sizeof(k.flags), h);
        h = Fnv1a(&k.generation, sizeof(k.generation), h);
        return (size_t)h;
    }
};

struct Plan {
    int algIndex = -1;        // index into the algorithm registry
    int devAlg = -1;          // DevAlg
    int nBlocks = 1;
    uint64_t chunkBytes = 0;  // bytes per loop of the sole executor (0 = whole message)
    uint32_t agreedFlags = 0; // buffer facts all ranks share for this call signature (what selection and execution used)
    uint64_t uses = 0;
};

class PlanCache {
public:
    static constexpr size_t kCapacity = 8192;
    bool Find(const PlanKey& k, Plan* out)
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = map_.find(k);
        if (it == map_.end()) { ++misses_; return false; }
        ++hits_;
        it->second.uses = ++tick_;
        *out = it->second;
        return true;
    }
    void Insert(const PlanKey& k, Plan p)
    {
        std::lock_guard<std::mutex> lk(mu_);
        if (map_.size() >= kCapacity) EvictLocked();
        p.uses = ++tick_;
        map_[k] = p;
    }
    void Clear()
    {
        std::lock_guard<std::mutex> lk(mu_);
        map_.clear();
    }
    size_t size() const { std::lock_guard<std::mutex> lk(mu_); return map_.size(); }
    uint64_t hits() const { return hits_; }
    uint64_t misses() const { return misses_; }

private:
    // drop the least recently used fifth (the reference evicts 20 % of its ring)
    void EvictLocked()
    {
        std::vector<uint64_t> ticks;
        ticks.reserve(map_.size());
        for (auto& kv : map_) ticks.push_back(kv.second.uses);
        size_t cut = ticks.size() / 5;
        std::nth_element(ticks.begin(), ticks.begin() + (long)cut, ticks.end());
        const uint64_t threshold = ticks[cut];
        for (auto it = map_.begin(); it != map_.end();) {
            if (it->second.uses <= threshold) it = map_.erase(it); else ++it;
        }
    }
    mutable std::mutex mu_;
    std::unordered_map<PlanKey, Plan, PlanKeyHash> map_;
    uint64_t tick_ = 0, hits_ = 0, misses_ = 0;
};

}  // namespace hccl
