#include "pool.hpp"

#include <algorithm>
#include <cstdio>

namespace tsw {
namespace {

inline uint64_t pow2_ceil(uint64_t v) {
    uint64_t r = 1;
    while (r < v) r <<= 1;
    return r;
}

// One 128 MiB chunk carved into equal slots: 64 x 2 MiB ("regular", serves the
// 2 MiB and 20 MiB request sizes) or 8 x 16 MiB ("irregular", serves requests
// rounded up to a power of two).  Bit i of free_mask = slot i is free.
// Follows Block in block_manager.hpp:38-125.
struct Chunk {
    uint64_t base = 0;       // phys
    bool regular = true;
    uint64_t avail = kChunkBytes;
    uint64_t free_mask = 0;
    int slots = 0;

    Chunk(uint64_t b, bool reg) : base(b), regular(reg) {
        slots = reg ? (int)(kChunkBytes / kRegular2MiB) : (int)(kChunkBytes / kIrregularSlot);
        free_mask = slots == 64 ? ~0ull : ((1ull << slots) - 1);
    }
    uint64_t slot_bytes() const { return regular ? kRegular2MiB : kIrregularSlot; }

    static void shape(bool regular, uint64_t size, uint64_t* round, int* step) {
        if (regular) {
            *round = size;
            *step = (int)(size / kRegular2MiB);
        } else {
            *round = pow2_ceil(size);
            *step = (int)(*round / kIrregularSlot);
        }
    }

    // try_acquire_block (:58-105): probe NON-OVERLAPPING windows of `step`
    // slots from the chunk start and take the first window that is entirely
    // free.  A window that would run past the last slot does not fit.
    // Divergence from the reference, on purpose: an irregular request of 8 MiB
    // or less has step 0 there, which returns the chunk base without marking
    // any slot (so two such requests overlap); here it takes one whole slot.
    uint64_t try_acquire(uint64_t size) {
        uint64_t round;
        int step;
        shape(regular, size, &round, &step);
        if (step == 0) { step = 1; round = slot_bytes(); }
        for (int s = 0; s + step <= slots; s += step) {
            uint64_t window = (step == 64 ? ~0ull : ((1ull << step) - 1)) << s;
            if ((free_mask & window) == window) {
                free_mask &= ~window;
                avail -= round;
                return base + (uint64_t)s * slot_bytes();
            }
        }
        return 0;
    }

    // release_block (:107-121)
    bool release(uint64_t ptr, uint64_t size) {
        uint64_t round;
        int step;
        shape(regular, size, &round, &step);
        if (ptr < base || ptr >= base + kChunkBytes || (ptr - base) % slot_bytes() != 0) return false;
        if (!regular && size == kRegular2MiB) {
            // A 2 MiB block is never taken from an irregular chunk; it can only be released into one
            // when the same address has been granted by two chunk objects over one 128 MiB and the
            // later grant owns the map entry.  The reference's zero step then flips no slot and only
            // adds the 2 MiB to the chunk's free bytes (:108-120); so does this.
            avail += size;
            return true;
        }
        if (step == 0) { step = 1; round = slot_bytes(); }
        int s = (int)((ptr - base) / slot_bytes());
        for (int i = 0; i < step && s + i < slots; ++i) free_mask |= 1ull << (s + i);
        avail += round;
        return true;
    }
};

// Max-heap of chunk ids by free bytes, driven by the standard heap algorithms
// exactly as sp_priority_queue is (:134-162): ties are broken the same way.
struct ChunkHeap {
    std::vector<int> c;
    const std::vector<Chunk>* chunks = nullptr;
    bool less(int a, int b) const { return (*chunks)[a].avail < (*chunks)[b].avail; }
    size_t size() const { return c.size(); }
    int top() const { return c.front(); }
    void push(int id) {
        c.push_back(id);
        std::push_heap(c.begin(), c.end(), [this](int a, int b) { return less(a, b); });
    }
    void pop() {
        std::pop_heap(c.begin(), c.end(), [this](int a, int b) { return less(a, b); });
        c.pop_back();
    }
    // The reference removes the first entry that *equals* the chunk, and its chunks compare by base
    // address (block_manager.hpp:124,155-161).  That matters when a retired chunk object is still
    // listed somewhere and a new one has since been made over the same 128 MiB: the entry removed is
    // the first with that base, not necessarily the object asked for.
    void remove(int id) {
        const uint64_t base = (*chunks)[id].base;
        auto it = std::find_if(c.begin(), c.end(), [&](int other) { return (*chunks)[other].base == base; });
        if (it != c.end()) {
            c.erase(it);
            std::make_heap(c.begin(), c.end(), [this](int a, int b) { return less(a, b); });
        }
    }
};

class BuddyPool : public Pool {
public:
    BuddyPool(uint64_t total_budget, int server_id, DeviceMemory* mem)
        : budget_(total_budget), canon_(server_id), mem_(mem) {
        regular_heap_.chunks = &chunks_;
        irregular_heap_.chunks = &chunks_;
    }

    ~BuddyPool() override {
        if (base_) mem_->release(base_);
        for (auto& kv : oversize_idle_)
            for (auto& a : kv.second) mem_->release(a.phys);
        for (auto& kv : oversize_live_) mem_->release(kv.first);
    }

    // init_allocation (:264-273): floor(budget / 128 MiB) chunks, pushed in
    // allocation order onto the LIFO free list.  One allocation backs them all.
    int init() override {
        n_chunks_ = budget_ / kChunkBytes;
        canon_base_ = canon_.bump(n_chunks_ * kChunkBytes);
        if (n_chunks_ == 0) return 0;
        if (mem_->plan_only()) base_ = canon_base_;
        else if (mem_->alloc(n_chunks_ * kChunkBytes, &base_) != 0) return -1;
        for (uint64_t i = 0; i < n_chunks_; ++i) free_chunks_.push_back(base_ + i * kChunkBytes);
        return 0;
    }

    uint64_t pool_base() const override { return base_; }
    uint64_t pool_chunks() const override { return n_chunks_; }

    uint64_t canon_of(uint64_t phys) const override {
        if (phys >= base_ && phys < base_ + n_chunks_ * kChunkBytes) return canon_base_ + (phys - base_);
        auto it = oversize_live_.find(phys);
        return it == oversize_live_.end() ? 0 : it->second.canon;
    }

    uint64_t canon_inside(uint64_t phys) const override {
        if (phys >= base_ && phys < base_ + n_chunks_ * kChunkBytes) return canon_base_ + (phys - base_);
        for (auto& kv : oversize_live_)
            if (phys >= kv.first && phys < kv.first + kv.second.size) return kv.second.canon + (phys - kv.first);
        return 0;
    }

    void regions(std::vector<std::pair<uint64_t, uint64_t>>* out) const override {
        if (mem_->plan_only()) return;
        if (base_) out->emplace_back(base_, n_chunks_ * kChunkBytes);
        for (auto& kv : oversize_live_) out->emplace_back(kv.first, kv.second.size);
        for (auto& kv : oversize_idle_)
            for (auto& a : kv.second) out->emplace_back(a.phys, a.size);
    }

    // acquire_block (:288-301)
    int acquire(uint64_t size, bool, DevAddr* out) override {
        if (size == kRegular2MiB || size == kRegular20MiB) return acquire_class(size, true, out);
        if (size <= kChunkBytes) return acquire_class(size, false, out);
        // Larger than a chunk.  The reference leaves the pool here with a raw
        // cudaMalloc ("expect this never happens") and loses the block on
        // evict (:295-300,402-404).  Same placement -- outside the pool, one
        // canonical address per acquisition -- but blocks are kept on a
        // per-size idle list when evicted and reused.
        DevAddr a;
        a.canon = canon_.bump(size);
        auto& idle = oversize_idle_[size];
        if (mem_->plan_only()) {
            a.phys = a.canon;  // nothing to reuse: a plan has addresses only
        } else if (!idle.empty()) {
            a.phys = idle.back().phys;
            idle.pop_back();
        } else if (mem_->alloc(size, &a.phys) != 0) {
            return -1;
        }
        a.size = size;
        oversize_live_[a.phys] = a;
        *out = a;
        return 0;
    }

    // evict_block (:382-405)
    int evict(uint64_t phys, uint64_t size, bool) override {
        auto it = owner_.find(phys);
        if (it != owner_.end()) {
            int id = it->second;
            chunks_[id].release(phys, size);
            if (size == kRegular2MiB || size == kRegular20MiB) {
                if (std::find(deactive_regular_.begin(), deactive_regular_.end(), id) == deactive_regular_.end()) {
                    deactive_regular_.push_back(id);
                    regular_heap_.remove(id);
                }
            } else if (size <= kChunkBytes) {
                if (std::find(deactive_irregular_.begin(), deactive_irregular_.end(), id) == deactive_irregular_.end()) {
                    deactive_irregular_.push_back(id);
                    irregular_heap_.remove(id);
                }
            }
            held_[id]--;
            owner_.erase(it);
            return 0;
        }
        auto ov = oversize_live_.find(phys);
        if (ov != oversize_live_.end()) {
            if (!mem_->plan_only()) oversize_idle_[size].push_back(ov->second);
            oversize_live_.erase(ov);
            return 0;
        }
        last_warning = "cannot find physical block for ptr";
        return 1;
    }

    // finish_block_alloc (:275-286)
    void finish_block_alloc() override {
        for (int id : active_regular_) regular_heap_.push(id);
        active_regular_.clear();
        for (int id : active_irregular_) irregular_heap_.push(id);
        active_irregular_.clear();
    }

    // finish_release_block (:355-380)
    void finish_release_block() override {
        for (int id : deactive_regular_) {
            if (chunks_[id].avail == kChunkBytes) retire(id);
            else regular_heap_.push(id);
        }
        deactive_regular_.clear();
        for (int id : deactive_irregular_) {
            if (chunks_[id].avail == kChunkBytes) retire(id);
            else irregular_heap_.push(id);
        }
        deactive_irregular_.clear();
    }

private:
    // acquire_block_temp (:303-353)
    int acquire_class(uint64_t size, bool regular, DevAddr* out) {
        std::vector<int>& active = regular ? active_regular_ : active_irregular_;
        ChunkHeap& heap = regular ? regular_heap_ : irregular_heap_;
        for (int id : active) {
            uint64_t p = chunks_[id].try_acquire(size);
            if (p) return granted(p, id, out);
        }
        while (heap.size() > 0 && chunks_[heap.top()].avail >= size) {
            int id = heap.top();
            active.push_back(id);
            heap.pop();
            uint64_t p = chunks_[id].try_acquire(size);
            if (p) return granted(p, id, out);
        }
        if (free_chunks_.empty()) {
            last_warning = "no free physical block";
            return -1;
        }
        int id = new_chunk(free_chunks_.back(), regular);
        free_chunks_.pop_back();
        active.push_back(id);
        uint64_t p = chunks_[id].try_acquire(size);
        if (!p) {
            last_warning = "cannot acquire block from a free physical block";
            return -1;
        }
        return granted(p, id, out);
    }

    int granted(uint64_t p, int id, DevAddr* out) {
        auto prev = owner_.find(p);
        if (prev != owner_.end()) held_[prev->second]--;   // the same address granted again: the entry changes hands
        owner_[p] = id;
        held_[id]++;
        out->phys = p;
        out->canon = canon_base_ + (p - base_);
        return 0;
    }

    // Chunk objects live as long as anything refers to them, as the reference's shared pointers do:
    // a list, a heap, or an address that was granted from them and has not been released yet.
    bool referenced(int id) const {
        auto in = [id](const std::vector<int>& v) { return std::find(v.begin(), v.end(), id) != v.end(); };
        return held_[id] > 0 || in(active_regular_) || in(active_irregular_) || in(deactive_regular_) ||
               in(deactive_irregular_) || in(regular_heap_.c) || in(irregular_heap_.c);
    }

    int new_chunk(uint64_t base, bool regular) {
        // ids of retired chunks are reused once nothing refers to them any more
        for (size_t k = 0; k < retired_.size(); ++k) {
            const int id = retired_[k];
            if (!referenced(id)) {
                retired_.erase(retired_.begin() + (long)k);
                chunks_[id] = Chunk(base, regular);
                return id;
            }
        }
        chunks_.emplace_back(base, regular);
        held_.push_back(0);
        return (int)chunks_.size() - 1;
    }

    void retire(int id) {
        free_chunks_.push_back(chunks_[id].base);
        if (std::find(retired_.begin(), retired_.end(), id) == retired_.end()) retired_.push_back(id);
    }

    uint64_t budget_;
    CanonSpace canon_;
    DeviceMemory* mem_;
    uint64_t base_ = 0, canon_base_ = 0, n_chunks_ = 0;

    std::vector<uint64_t> free_chunks_;  // LIFO: back() is taken first
    std::vector<Chunk> chunks_;
    std::vector<int> retired_;           // ids whose 128 MiB went back to the free list; reusable once unreferenced
    std::vector<int> held_;              // per chunk id: granted addresses that still map to it in owner_
    std::vector<int> active_regular_, deactive_regular_, active_irregular_, deactive_irregular_;
    ChunkHeap regular_heap_, irregular_heap_;
    std::unordered_map<uint64_t, int> owner_;  // granted address -> chunk id (requested_to_block_map_)

    std::map<uint64_t, std::vector<DevAddr>> oversize_idle_;
    std::unordered_map<uint64_t, DevAddr> oversize_live_;
};

// FixedSizeBlockManager (:188-258): per-size LIFO free lists over raw device
// allocations with a byte budget; selected by BLOCK_MANAGER=Fixed.
class FixedPool : public Pool {
public:
    FixedPool(uint64_t total_budget, int server_id, DeviceMemory* mem)
        : budget_(total_budget), canon_(server_id), mem_(mem) {}

    ~FixedPool() override {
        for (auto& kv : live_) mem_->release(kv.first);
    }

    int init() override { return 0; }

    uint64_t canon_of(uint64_t phys) const override {
        auto it = live_.find(phys);
        return it == live_.end() ? 0 : it->second.canon;
    }
    uint64_t canon_inside(uint64_t phys) const override {
        for (auto& kv : live_)
            if (phys >= kv.first && phys < kv.first + kv.second.size) return kv.second.canon + (phys - kv.first);
        return 0;
    }

    void regions(std::vector<std::pair<uint64_t, uint64_t>>* out) const override {
        if (mem_->plan_only()) return;
        for (auto& kv : live_) out->emplace_back(kv.first, kv.second.size);
    }

    int acquire(uint64_t size, bool external_call, DevAddr* out) override {
        auto& idle = idle_[size];
        if (!idle.empty()) {
            out->phys = idle.back();
            idle.pop_back();
            out->canon = live_[out->phys].canon;
            return 0;
        }
        if (budget_ < size) {
            // free idle blocks, largest size first, until the request fits (:205-221)
            for (auto& kv : idle_) {
                while (!kv.second.empty()) {
                    uint64_t p = kv.second.back();
                    kv.second.pop_back();
                    mem_->release(p);
                    live_.erase(p);
                    budget_ += kv.first;
                    if (budget_ >= size) break;
                }
                if (budget_ >= size) break;
            }
        }
        int rc = raw_alloc(size, out);
        if (rc != 0) return rc;
        if (budget_ >= size) budget_ -= size;
        else if (!external_call) last_warning = "no enough memory when acquiring block";  // (:232-238) over budget
        return 0;
    }

    int evict(uint64_t phys, uint64_t size, bool free_flag) override {
        if (free_flag) {
            mem_->release(phys);
            live_.erase(phys);
            budget_ += size;
        } else {
            idle_[size].push_back(phys);
        }
        return 0;
    }

private:
    int raw_alloc(uint64_t size, DevAddr* out) {
        out->canon = canon_.bump(size);
        if (mem_->plan_only()) out->phys = out->canon;
        else if (mem_->alloc(size, &out->phys) != 0) return -1;
        out->size = size;
        live_[out->phys] = *out;
        return 0;
    }

    uint64_t budget_;
    CanonSpace canon_;
    DeviceMemory* mem_;
    std::map<uint64_t, std::vector<uint64_t>, std::greater<uint64_t>> idle_;  // largest size first
    std::unordered_map<uint64_t, DevAddr> live_;  // by phys
};

}  // namespace

std::unique_ptr<Pool> make_buddy_pool(uint64_t total_budget, int server_id, DeviceMemory* mem) {
    return std::unique_ptr<Pool>(new BuddyPool(total_budget, server_id, mem));
}
std::unique_ptr<Pool> make_fixed_pool(uint64_t total_budget, int server_id, DeviceMemory* mem) {
    return std::unique_ptr<Pool>(new FixedPool(total_budget, server_id, mem));
}

}  // namespace tsw
