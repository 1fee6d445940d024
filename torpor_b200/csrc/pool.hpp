// Pooled GPU block allocator of the swap engine.
//
// Makes, decision for decision, the placements of the reference's
// BuddyBasedBlockManager / FixedSizeBlockManager
// (include/server/block_manager.hpp:188-418) but on flat state: every 128 MiB
// chunk is one bitmask of slots instead of an ordered map, chunks are indices
// into one array, and the whole pool is ONE device allocation so that a single
// IPC handle / peer mapping covers it.
//
// Addresses come in two flavours.  `phys` is where the bytes live.  `canon` is
// the same location in a canonical address space that starts at a fixed base
// for every run: tables whose iteration order depends on address hashing are
// keyed by canon so that block request order is reproducible.
#ifndef TORPOR_SWAP_POOL_HPP_
#define TORPOR_SWAP_POOL_HPP_

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

namespace tsw {

constexpr uint64_t kMiB = 1ull << 20;
constexpr uint64_t kChunkBytes = 128 * kMiB;        // block_manager.hpp:23
constexpr uint64_t kRegular2MiB = 2 * kMiB;         // :28
constexpr uint64_t kRegular20MiB = 20 * kMiB;       // :29
constexpr uint64_t kIrregularSlot = 16 * kMiB;      // :30
constexpr uint64_t kHiddenBudget = 5ull << 30;      // memory_manager.hpp:43-44
constexpr uint64_t kCanonBase = 0x600000000000ull;  // canonical device VA of server 0
constexpr uint64_t kCanonStride = 0x010000000000ull;
constexpr uint64_t kDevAllocAlign = 2 * kMiB;

struct DevAddr {
    uint64_t phys = 0;
    uint64_t canon = 0;
    uint64_t size = 0;  // filled for allocations outside the chunked pool
};

// Source of raw device memory: the CUDA runtime, or (plan-only engines) nothing
// at all -- then phys == canon and no byte ever moves.
class DeviceMemory {
public:
    virtual ~DeviceMemory() {}
    virtual int alloc(uint64_t size, uint64_t* phys) = 0;  // 0 on success
    virtual int release(uint64_t phys) = 0;
    virtual bool plan_only() const = 0;
};

// Hands out canonical addresses the way a 2 MiB-aligned bump allocator over a
// fresh address space would, and remembers canon <-> phys for everything that
// is not inside the pool.
class CanonSpace {
public:
    explicit CanonSpace(int server_id) : base_(kCanonBase + (uint64_t)server_id * kCanonStride) {}
    uint64_t base() const { return base_; }
    uint64_t bump(uint64_t size) {
        uint64_t c = base_ + next_;
        next_ += (size + kDevAllocAlign - 1) / kDevAllocAlign * kDevAllocAlign;
        return c;
    }
private:
    uint64_t base_;
    uint64_t next_ = 0;
};

class Pool {
public:
    virtual ~Pool() {}
    virtual int init() = 0;
    // acquire_block(ptr, size, external_call) -- block_manager.hpp:173
    virtual int acquire(uint64_t size, bool external_call, DevAddr* out) = 0;
    // evict_block(ptr, size, free_flag) -- :174
    virtual int evict(uint64_t phys, uint64_t size, bool free_flag) = 0;
    virtual void finish_block_alloc() {}     // :176
    virtual void finish_release_block() {}   // :177
    virtual uint64_t pool_base() const { return 0; }
    virtual uint64_t pool_chunks() const { return 0; }
    // canon of an address this pool handed out (0 if unknown)
    virtual uint64_t canon_of(uint64_t phys) const = 0;
    // canon of any address inside a block this pool currently has handed out (0 if unknown)
    virtual uint64_t canon_inside(uint64_t phys) const = 0;
    // every device allocation this pool holds, as (base, bytes): what another process has to
    // map to reach any block the pool can hand out
    virtual void regions(std::vector<std::pair<uint64_t, uint64_t>>* out) const = 0;
    std::string last_warning;
};

std::unique_ptr<Pool> make_buddy_pool(uint64_t total_budget, int server_id, DeviceMemory* mem);
std::unique_ptr<Pool> make_fixed_pool(uint64_t total_budget, int server_id, DeviceMemory* mem);

}  // namespace tsw
#endif
