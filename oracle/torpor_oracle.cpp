// TEST INFRASTRUCTURE ONLY -- never linked into, imported by or executed from the
// shipped library.  CPU restatement of Torpor's model-swap path, used as the
// checker in tests, in the smoke check and as the benchmark's CPU baseline.
//
// Each section restates, in plain single-threaded C++, the algorithm of one
// reference file and cites the lines it follows:
//   pool of 128 MiB chunks       include/server/block_manager.hpp
//   model tables                 include/server/model_repo.hpp
//   manager (swap-in / swap-out) include/server/memory_manager.hpp
//   eviction policy              include/server/evictor.hpp
//   swap scheduler               include/server/controller.hpp:296-389
// Parity is PINNED: tests/golden/ holds tables, victims and scheduling decisions
// produced by the reference's own headers compiled against a host-memory CUDA
// stand-in (ref_harness.cpp; controller.hpp with its socket and executor headers
// shadowed); this restatement reproduces them bit for bit
// (tests/test_oracle_golden.py, tests/test_scheduler.py).
//
// "Device" memory here is a label space: addresses start at the same canonical
// base as in the stand-in (0x600000000000 + 1 TiB per GPU), bytes live in a
// lazily committed backing mapping.  The reference's staging threads, transfer
// thread and event round trips are not modelled: a swap-in completes before
// swap_in() returns, which is the state the reference reaches once its last
// readiness group is published.

#include "tso_abi.h"

#include <sys/mman.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <list>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

using std::string;
typedef unsigned char byte;

const uint64_t kCanonBase = 0x600000000000ull;
const uint64_t kCanonStride = 0x010000000000ull;
const uint64_t kTwoMiB = 2ull << 20;
const int kMaxDev = 16;

// ---------------------------------------------------------------- fake device
struct Device {
    uint64_t bump = 0;
    byte* backing = nullptr;
    uint64_t backed = 0;
};
Device g_dev[kMaxDev];
const uint64_t kBackingSpan = 1ull << 39;  // 512 GiB of address space per device, committed on touch

uint64_t dev_malloc(int dev, uint64_t size) {
    Device& d = g_dev[dev];
    if (!d.backing) {
        void* p = mmap(nullptr, kBackingSpan, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
        if (p == MAP_FAILED) { perror("oracle backing"); abort(); }
        d.backing = (byte*)p;
    }
    uint64_t off = d.bump;
    d.bump += (size + kTwoMiB - 1) / kTwoMiB * kTwoMiB;
    if (d.bump > kBackingSpan) { fprintf(stderr, "oracle: device address space exhausted\n"); abort(); }
    return kCanonBase + (uint64_t)dev * kCanonStride + off;
}
// TORPOR_ORACLE_TABLES_ONLY=1: placement and tables only -- no parameter byte is stored or moved
// (payloads may then be null), so a 13.5 GB weight set can be held to its tables in a few MB.
bool tables_only() {
    const char* v = getenv("TORPOR_ORACLE_TABLES_ONLY");
    return v && v[0] == '1';
}
byte* dev_bytes(uint64_t addr) {
    int dev = (int)((addr - kCanonBase) / kCanonStride);
    return g_dev[dev].backing + (addr - kCanonBase - (uint64_t)dev * kCanonStride);
}
void dev_reset() {
    for (int i = 0; i < kMaxDev; ++i) {
        if (g_dev[i].backing) munmap(g_dev[i].backing, kBackingSpan);
        g_dev[i] = Device();
    }
}

// ---------------------------------------------------------------- pool (block_manager.hpp)
const uint64_t kChunk = 128ull << 20;       // :23
const uint64_t kReg2 = 2ull << 20;          // :28
const uint64_t kReg20 = 20ull << 20;        // :29
const uint64_t kIrrMin = 16ull << 20;       // :30

struct Chunk {                               // struct Block, :38-125
    uint64_t base;
    bool regular;
    uint64_t avail = kChunk;
    std::map<uint64_t, bool> slot_free;      // addr_status_map_

    Chunk(uint64_t b, bool reg) : base(b), regular(reg) {
        uint64_t s = reg ? kReg2 : kIrrMin;  // :45-56
        for (uint64_t i = 0; i < kChunk / s; ++i) slot_free[base + i * s] = true;
    }
    uint64_t try_acquire(uint64_t size) {    // :58-105
        uint64_t round = regular ? size : (uint64_t)std::pow(2, std::ceil(std::log2((double)size)));
        uint64_t step = regular ? size / kReg2 : round / kIrrMin;
        auto it = slot_free.begin();
        while (it != slot_free.end()) {
            bool ok = true;
            for (uint64_t i = 0; i < step; ++i) {
                if (it == slot_free.end()) { ok = false; break; }
                if (!it->second) ok = false;
                ++it;
            }
            if (ok) {
                it = std::prev(it, (long)step);
                uint64_t got = it->first;
                for (uint64_t i = 0; i < step; ++i) { it->second = false; ++it; }
                avail -= round;
                return got;
            }
        }
        return 0;
    }
    void release(uint64_t ptr, uint64_t size) {  // :107-121
        uint64_t round = regular ? size : (uint64_t)std::pow(2, std::ceil(std::log2((double)size)));
        uint64_t step = regular ? round / kReg2 : round / kIrrMin;
        auto it = slot_free.find(ptr);
        if (it == slot_free.end()) return;
        for (uint64_t i = 0; i < step; ++i) { it->second = true; ++it; }
        avail += round;
    }
};
typedef std::shared_ptr<Chunk> ChunkP;

struct Heap {                                // sp_priority_queue, :134-162
    std::vector<ChunkP> c;
    static bool less(const ChunkP& a, const ChunkP& b) { return a->avail < b->avail; }
    void push(const ChunkP& x) { c.push_back(x); std::push_heap(c.begin(), c.end(), less); }
    void pop() { std::pop_heap(c.begin(), c.end(), less); c.pop_back(); }
    void remove(const ChunkP& x) {
        auto it = std::find_if(c.begin(), c.end(), [&](const ChunkP& y) { return x->base == y->base; });
        if (it != c.end()) { c.erase(it); std::make_heap(c.begin(), c.end(), less); }
    }
};

struct PoolBase {
    virtual ~PoolBase() {}
    virtual void init() {}
    virtual uint64_t acquire(uint64_t size, bool external) = 0;
    virtual void evict(uint64_t ptr, uint64_t size) = 0;
    virtual void finish_alloc() {}
    virtual void finish_release() {}
    int dev = 0;
    uint64_t budget = 0;
    std::vector<uint64_t> chunks;
};

struct BuddyPool : PoolBase {                // BuddyBasedBlockManager, :260-418
    std::vector<uint64_t> free_pool;
    std::vector<ChunkP> act_reg, deact_reg, act_irr, deact_irr;
    Heap heap_reg, heap_irr;
    std::unordered_map<uint64_t, ChunkP> owner;

    void init() override {                   // :264-273
        for (uint64_t i = 0; i < budget / kChunk; ++i) free_pool.push_back(dev_malloc(dev, kChunk));
        chunks = free_pool;
    }
    void finish_alloc() override {           // :275-286
        for (auto& b : act_reg) heap_reg.push(b);
        act_reg.clear();
        for (auto& b : act_irr) heap_irr.push(b);
        act_irr.clear();
    }
    uint64_t acquire(uint64_t size, bool) override {  // :288-301
        if (size == kReg2 || size == kReg20) return from_class(size, act_reg, heap_reg, true);
        if (size <= kChunk) return from_class(size, act_irr, heap_irr, false);
        return dev_malloc(dev, size);        // raw allocation outside the pool
    }
    uint64_t from_class(uint64_t size, std::vector<ChunkP>& act, Heap& heap, bool reg) {  // :303-353
        for (auto& b : act) {
            uint64_t p = b->try_acquire(size);
            if (p) { owner[p] = b; return p; }
        }
        while (!heap.c.empty() && heap.c.front()->avail >= size) {
            act.push_back(heap.c.front());
            heap.pop();
            uint64_t p = act.back()->try_acquire(size);
            if (p) { owner[p] = act.back(); return p; }
        }
        if (free_pool.empty()) { fprintf(stderr, "oracle: no free physical block\n"); exit(1); }
        act.push_back(std::make_shared<Chunk>(free_pool.back(), reg));
        free_pool.pop_back();
        uint64_t p = act.back()->try_acquire(size);
        if (!p) { fprintf(stderr, "oracle: cannot acquire from a free physical block\n"); exit(1); }
        owner[p] = act.back();
        return p;
    }
    void finish_release() override {         // :355-380
        for (auto& b : deact_reg) {
            if (b->avail == kChunk) free_pool.push_back(b->base);
            else heap_reg.push(b);
        }
        deact_reg.clear();
        for (auto& b : deact_irr) {
            if (b->avail == kChunk) free_pool.push_back(b->base);
            else heap_irr.push(b);
        }
        deact_irr.clear();
    }
    void evict(uint64_t ptr, uint64_t size) override {  // :382-405
        auto it = owner.find(ptr);
        if (it == owner.end()) return;       // a raw allocation: the reference reports and forgets it
        ChunkP b = it->second;
        b->release(ptr, size);
        auto listed = [&](std::vector<ChunkP>& v) {
            return std::find_if(v.begin(), v.end(), [&](const ChunkP& x) { return x.get() == b.get(); }) != v.end();
        };
        if (size == kReg2 || size == kReg20) {
            if (!listed(deact_reg)) { deact_reg.push_back(b); heap_reg.remove(b); }
        } else if (size <= kChunk) {
            if (!listed(deact_irr)) { deact_irr.push_back(b); heap_irr.remove(b); }
        }
        owner.erase(ptr);
    }
};

struct FixedPool : PoolBase {                // FixedSizeBlockManager, :188-258
    std::map<uint64_t, std::vector<uint64_t>, std::greater<uint64_t>> idle;
    uint64_t acquire(uint64_t size, bool) override {  // :192-242
        auto& v = idle[size];
        if (!v.empty()) { uint64_t p = v.back(); v.pop_back(); return p; }
        if (budget < size) {
            for (auto& kv : idle) {
                while (!kv.second.empty()) {
                    kv.second.pop_back();
                    budget += kv.first;
                    if (budget >= size) break;
                }
                if (budget >= size) break;
            }
        }
        if (budget >= size) budget -= size;
        return dev_malloc(dev, size);
    }
    void evict(uint64_t ptr, uint64_t size) override { idle[size].push_back(ptr); }  // :244-254
};

// ---------------------------------------------------------------- tables (model_repo.hpp)
struct BlockInfo { uint64_t size = 0; bool is_model = false; std::unordered_set<uint64_t> ephe; };       // :12-17
struct ModelBlock { byte* host = nullptr; std::unordered_set<uint64_t> params; };                        // :19-23
struct ParamInfo { uint64_t size = 0; byte* host = nullptr; };                                           // :25-30
struct HostModel {                                                                                       // :37-46
    std::unordered_map<void*, BlockInfo> blocks;           // pointer-keyed on purpose: same hashing as the reference
    std::unordered_map<uint64_t, uint64_t> data_block;
    std::unordered_map<uint64_t, ModelBlock> model_blocks;
    std::unordered_map<uint64_t, ParamInfo> params;
    uint64_t total = 0;
};
struct BlockDev { bool in_cuda = false, in_pin = false; uint64_t cuda = 0; };                            // :48-53
struct ParamDev { uint64_t cuda = 0; };
struct DevModel { std::unordered_map<uint64_t, BlockDev> blocks; std::unordered_map<uint64_t, ParamDev> params; int status = 1; };

struct Repo {
    std::unordered_map<string, std::vector<uint64_t>> access_order;
    std::unordered_map<string, HostModel> host;
    std::unordered_map<int, std::unordered_map<string, DevModel>> dev;
    std::unordered_map<string, std::unordered_set<int>> active;   // model_active_device_map_ (model_repo.hpp:185)
};
Repo g_repo;

// ---------------------------------------------------------------- manager (memory_manager.hpp)
enum { kHost = 0, kPinned = 1, kCuda = 2 };

struct Manager {
    int id = 0;
    std::unique_ptr<PoolBase> pool;
    bool tracking = false;
    string track_func;
    std::unordered_map<string, std::unordered_map<uint64_t, std::pair<int, uint64_t>>> ready;
    std::unordered_set<uint64_t> active_params;

    void init_readiness(const string& f, int flag) {                 // :234-238
        for (auto& kv : g_repo.host[f].params) ready[f].emplace(kv.first, std::make_pair(flag, kv.first));
    }

    uint64_t do_malloc(const string& f, uint64_t size, bool is_model) {  // :85-94 + model_repo.hpp:133-141
        uint64_t p = pool->acquire(size, true);
        HostModel& h = g_repo.host[f];
        if (is_model) h.model_blocks[p] = ModelBlock{(byte*)malloc(size ? size : 1), {}};
        h.blocks[(void*)p] = BlockInfo{size, is_model, {}};
        h.total += size;
        g_repo.dev[id][f].blocks[p] = BlockDev{true, false, p};
        return p;
    }

    int upload(const string& f, uint64_t dst, const void* payload, uint64_t size) {  // :124-142 + model_repo.hpp:151-168
        HostModel& h = g_repo.host[f];
        for (auto& kv : h.model_blocks) {
            uint64_t b = kv.first;
            if (dst >= b && dst < b + h.blocks[(void*)b].size) {
                byte* host = kv.second.host + (dst - b);
                kv.second.params.insert(dst);
                if (!tables_only()) memcpy(host, payload, size);
                h.params[dst] = ParamInfo{size, host};
                h.data_block[dst] = b;
                g_repo.dev[id][f].params[dst] = ParamDev{dst};
                if (!tables_only()) memcpy(dev_bytes(dst), payload, size);
                return 0;
            }
        }
        return -1;
    }

    void do_free(const string& f, uint64_t p) {                      // :97-110 + model_repo.hpp:144-149
        DevModel& d = g_repo.dev[id][f];
        if (!d.blocks.count(p)) return;
        HostModel& h = g_repo.host[f];
        if (h.blocks[(void*)p].is_model) return;
        if (d.blocks[p].in_cuda) pool->evict(d.blocks[p].cuda, h.blocks[(void*)p].size);
        for (uint64_t e : h.blocks[(void*)p].ephe) h.data_block.erase(e);
        h.blocks.erase((void*)p);
    }

    bool mark_access(uint64_t p) {                                   // :273-284 + model_repo.hpp:102-109
        if (!tracking) return true;
        if (!g_repo.host[track_func].params.count(p)) return false;
        auto& order = g_repo.access_order[track_func];
        if (std::find(order.begin(), order.end(), p) == order.end()) order.push_back(p);
        return true;
    }

    void place(const string& f) {                                    // check_and_malloc_model, :451-507
        HostModel& h = g_repo.host[f];
        if (!g_repo.dev[id].count(f)) g_repo.dev[id][f] = DevModel{{}, {}, 3};
        if (!ready.count(f)) init_readiness(f, kHost);
        DevModel& d = g_repo.dev[id][f];
        for (auto& kv : h.blocks) {
            uint64_t b = (uint64_t)kv.first;
            if (d.blocks.count(b) && d.blocks[b].in_cuda) continue;
            d.blocks[b].cuda = pool->acquire(kv.second.size, false);
            d.blocks[b].in_cuda = true;
            if (kv.second.is_model)
                for (uint64_t p : h.model_blocks[b].params) d.params[p].cuda = p - b + d.blocks[b].cuda;  // :477-479
        }
        active_params.clear();
        for (uint64_t p : g_repo.access_order[f]) active_params.insert(p);
        pool->finish_alloc();
    }

    void swap_in(const string& f, int src) {                         // sig_trans_thread :213-227 + transfer_model :331-438
        if (!g_repo.host.count(f)) return;
        if (src >= 0 && (!g_repo.dev[src].count(f) || g_repo.dev[src][f].status != 0)) src = -1;
        place(f);
        HostModel& h = g_repo.host[f];
        DevModel& d = g_repo.dev[id][f];
        for (uint64_t p : g_repo.access_order[f]) {
            auto r = ready[f].find(p);
            if (r == ready[f].end() || r->second.first == kCuda) continue;
            const byte* from = src < 0 ? h.params[p].host : dev_bytes(g_repo.dev[src][f].params[p].cuda);
            if (!tables_only()) memcpy(dev_bytes(d.params[p].cuda), from, h.params[p].size);   // :389-396
            r->second = std::make_pair((int)kCuda, d.params[p].cuda);      // :445
        }
    }

    void evict(const string& f) {                                    // :240-259
        if (!ready.count(f)) return;
        HostModel& h = g_repo.host[f];
        DevModel& d = g_repo.dev[id][f];
        for (auto& kv : h.blocks) {
            uint64_t b = (uint64_t)kv.first;
            if (!d.blocks[b].in_cuda) continue;
            d.blocks[b].in_cuda = false;
            pool->evict(d.blocks[b].cuda, kv.second.size);
            if (kv.second.is_model)
                for (uint64_t p : h.model_blocks[b].params) {        // reset_model_readiness, :301-309
                    auto r = ready[f].find(p);
                    if (r != ready[f].end()) r->second = std::make_pair(d.blocks[b].in_pin ? (int)kPinned : (int)kHost, (uint64_t)0);
                }
        }
        pool->finish_release();
    }

    bool cache_interior(const string& f, uint64_t a) {               // model_repo.hpp:111-122
        HostModel& h = g_repo.host[f];
        if (h.data_block.count(a)) return true;
        for (auto& kv : h.blocks) {
            uint64_t b = (uint64_t)kv.first;
            if (a >= b && a < b + kv.second.size) {
                h.data_block[a] = b;
                kv.second.ephe.insert(a);
                return true;
            }
        }
        return false;
    }

    uint64_t phy(const string& f, uint64_t p, bool amid) {           // get_phy_address, :542-568
        if (!g_repo.host.count(f)) return p;
        HostModel& h = g_repo.host[f];
        if (!h.data_block.count(p)) {
            if (amid) cache_interior(f, p);                          // valid_memory_address answers false, :293-298
            return p;
        }
        BlockDev& b = g_repo.dev[id][f].blocks[h.data_block[p]];
        if (b.in_cuda && b.cuda) return p - h.data_block[p] + b.cuda;
        return p;
    }

    uint64_t translate(const string& f, uint64_t p) {                // get_cuda_addr :261-271, check_param_readiness :527-540
        if (!g_repo.dev[id].count(f)) return p;
        if (!g_repo.host[f].params.count(p)) return phy(f, p, true);
        if (!ready.count(f)) return p;
        if (active_params.count(p) && ready[f].count(p)) return ready[f][p].second;
        return g_repo.dev[id][f].params[p].cuda;
    }

    bool alloc_ok(const string& f) {                                 // :195-210
        if (!g_repo.host.count(f)) return false;
        if (!g_repo.dev[id].count(f)) return false;
        DevModel& d = g_repo.dev[id][f];
        for (auto& kv : g_repo.host[f].blocks) {
            uint64_t b = (uint64_t)kv.first;
            if (!d.blocks.count(b) || !d.blocks[b].in_cuda) return false;
        }
        return true;
    }
};

// ---------------------------------------------------------------- eviction policy (evictor.hpp)
typedef std::list<std::pair<string, uint64_t>> Lru;

struct EvictorBase {
    virtual ~EvictorBase() {}
    virtual std::vector<string> add(int g, const string& f, uint64_t sz, std::unordered_map<string, int>& level) = 0;
    virtual void force(int g, const string& f) = 0;
    virtual void lock(int g, const string& f) = 0;
    void unlock(int g, const string& f) { locked[g].erase(f); }
    uint64_t budget = 0;
    std::vector<std::unordered_set<string>> locked;
    std::vector<uint64_t> cur;
    std::unordered_map<string, int> level;
};

struct LruEvictor : EvictorBase {            // :190-264
    std::vector<Lru> items;
    std::vector<std::unordered_map<string, Lru::iterator>> index;
    LruEvictor(int n, uint64_t b) { budget = b; items.resize(n); index.resize(n); locked.resize(n); cur.assign(n, 0); }
    std::vector<string> add(int g, const string& f, uint64_t sz, std::unordered_map<string, int>&) override {
        auto it = index[g].find(f);
        if (it != index[g].end()) { items[g].splice(items[g].begin(), items[g], it->second); return {}; }
        std::vector<string> out;
        while (cur[g] + sz >= budget) {
            bool found = false;
            for (auto r = items[g].rbegin(); r != items[g].rend(); ++r) {
                if (!locked[g].count(r->first)) {
                    out.push_back(r->first);
                    cur[g] -= r->second;
                    index[g].erase(r->first);
                    items[g].erase(std::next(r).base());
                    found = true;
                    break;
                }
            }
            if (!found) break;               // the reference would spin here; callers avoid the case
        }
        items[g].emplace_front(f, sz);
        index[g].emplace(f, items[g].begin());
        cur[g] += sz;
        return out;
    }
    void force(int g, const string& f) override {
        auto it = index[g].find(f);
        if (it == index[g].end()) return;
        cur[g] -= it->second->second;
        items[g].erase(it->second);
        index[g].erase(it);
    }
    void lock(int g, const string& f) override { if (index[g].count(f)) locked[g].insert(f); }
};

struct IaEvictor : EvictorBase {             // :28-188
    std::vector<Lru> first, second;
    std::vector<std::unordered_map<string, Lru::iterator>> ifirst, isecond;
    std::unordered_map<string, std::unordered_set<int>> homes;
    IaEvictor(int n, uint64_t b) {
        budget = b; first.resize(n); second.resize(n); ifirst.resize(n); isecond.resize(n); locked.resize(n); cur.assign(n, 0);
    }
    bool drop_lru(int g, Lru& l, std::unordered_map<string, Lru::iterator>& idx, std::vector<string>& out) {
        for (auto r = l.rbegin(); r != l.rend(); ++r) {
            if (!locked[g].count(r->first)) {
                out.push_back(r->first);
                cur[g] -= r->second;
                idx.erase(r->first);
                l.erase(std::next(r).base());
                return true;
            }
        }
        return false;
    }
    std::vector<string> add(int g, const string& f, uint64_t sz, std::unordered_map<string, int>& lv) override {
        if (homes.count(f) && homes[f].count(g)) {   // :43-60
            auto it = ifirst[g].find(f);
            if (it != ifirst[g].end()) first[g].splice(first[g].begin(), first[g], it->second);
            else {
                it = isecond[g].find(f);
                if (it != isecond[g].end()) second[g].splice(second[g].begin(), second[g], it->second);
            }
            return {};
        }
        std::vector<string> out;
        while (cur[g] + sz >= budget) if (!drop_lru(g, second[g], isecond[g], out)) break;   // :65-82
        while (cur[g] + sz >= budget) if (!drop_lru(g, first[g], ifirst[g], out)) break;     // :85-97 (spins in the reference)
        if (lv[f] >= 1 && homes[f].empty()) {                                               // :99-103
            first[g].emplace_front(f, sz);
            ifirst[g].emplace(f, first[g].begin());
        } else {                                                                            // :104-121
            second[g].emplace_front(f, sz);
            isecond[g].emplace(f, second[g].begin());
            if (lv[f] >= 1 && !homes[f].empty()) {
                for (int o : homes[f]) {
                    auto it = ifirst[o].find(f);
                    if (it != ifirst[o].end()) {
                        second[o].splice(second[o].begin(), first[o], it->second);
                        isecond[o].emplace(f, second[o].begin());
                        ifirst[o].erase(it);
                    }
                }
            }
        }
        homes[f].insert(g);
        cur[g] += sz;
        for (auto& m : out) {                                                               // :126-141
            homes[m].erase(g);
            if (lv[m] >= 1 && homes[m].size() == 1) {
                int o = *homes[m].begin();
                auto it = isecond[o].find(m);
                if (it != isecond[o].end()) {
                    first[o].splice(first[o].begin(), second[o], it->second);
                    ifirst[o].emplace(m, first[o].begin());
                    isecond[o].erase(it);
                }
            }
        }
        return out;
    }
    void force(int g, const string& f) override {                                           // :146-164
        auto it = ifirst[g].find(f);
        if (it != ifirst[g].end()) { cur[g] -= it->second->second; first[g].erase(it->second); ifirst[g].erase(it); }
        else {
            it = isecond[g].find(f);
            if (it != isecond[g].end()) { cur[g] -= it->second->second; second[g].erase(it->second); isecond[g].erase(it); }
        }
        homes[f].erase(g);
    }
    void lock(int g, const string& f) override { locked[g].insert(f); }                     // :166-168
};

// ---------------------------------------------------------------- swap scheduler (controller.hpp)
struct Sched {
    int n = 0;
    bool random_policy = false;
    std::vector<int> status;                 // executor_status_[i].status_ (:464)
    std::vector<int> pcie_pairs;             // pcie_pairs_ (:117)
    std::vector<std::vector<int>> nvlink;    // nvlink_topology_ (:118)
    std::unordered_map<string, int> level;   // model_level_map_

    static int level_to_status(int lv) { return (lv >= 0 && lv <= 2) ? lv + 2 : 3; }   // :26-33

    void decide(const string& f, int out[3]) {
        std::vector<int> avail;
        for (int i = 0; i < n; ++i) if (status[i] == -1) avail.push_back(i);
        if (avail.empty()) { out[0] = out[1] = out[2] = -1; return; }                    // :304-306,330-332
        if (g_repo.active.count(f) && !g_repo.active[f].empty()) {
            for (int g : g_repo.active[f])
                if (status[g] == -1) { out[0] = g; out[1] = -1; out[2] = 0; return; }   // :308-314,334-341
            if (!random_policy) {
                std::vector<int> src(g_repo.active[f].begin(), g_repo.active[f].end());  // :342-343
                int dst_gpu = avail[0], src_gpu = src[0];
                for (int gi : avail)
                    for (int gj : src)
                        if (nvlink[gi][gj] == 2) { dst_gpu = gi; src_gpu = gj; break; } // :345-355
                out[0] = dst_gpu; out[1] = src_gpu; out[2] = 1;                          // :375
                return;
            }
        }
        if (random_policy) {                                                              // :316-318
            out[0] = avail[rand() % avail.size()]; out[1] = -1; out[2] = level_to_status(level[f]);
            return;
        }
        int best = avail[0], best_status = status[pcie_pairs[avail[0]]];                  // :378-387
        for (int g : avail)
            if (status[pcie_pairs[g]] < best_status) { best_status = status[pcie_pairs[g]]; best = g; }
        out[0] = best; out[1] = -1; out[2] = level_to_status(level[f]);
    }
};

// ---------------------------------------------------------------- request handling (controller.hpp)
// The controller's loop body (:130-262) with its helpers (:271-294, :392-453), one event per
// call.  Signals to executors and acknowledgements to the router become lines of a trace:
// "S <gpu> <signal> <func>" and "A <ack> <resp>".
struct Ctrl {
    Sched sched;                                           // executor_status_, model_level_map_, schedule_func_
    std::unique_ptr<EvictorBase> ev;
    std::vector<string> running;                           // executor_status_[i].function_
    std::unordered_map<int, std::pair<int, string>> demand;   // executor_gpu_demand_ (:460)
    std::list<std::pair<string, bool>> waiting;            // req_queue_ (:466)
    int cur_id = 0;
    std::vector<string> trace;

    void send(const string& f, int gpu, int sig) { trace.push_back("S " + std::to_string(gpu) + " " + std::to_string(sig) + " " + f); }
    void ack(int gpu) { trace.push_back("A 0 " + std::to_string(gpu)); }                    // :432-440
    void add_info(const string& f, int gpu) { g_repo.dev[gpu][f].status = 0; g_repo.active[f].insert(gpu); }      // model_repo.hpp:82-85
    void remove_info(const string& f, int gpu) { g_repo.dev[gpu][f].status = 3; g_repo.active[f].erase(gpu); }    // model_repo.hpp:87-90

    int naive() {                                                                            // :271-281
        for (int i = 0; i < sched.n; ++i) if (sched.status[i] == -1) return i;
        return -1;
    }
    int placement() {                                                                        // :283-294
        int g = -1;
        if (sched.status[cur_id] == -1) { g = cur_id; cur_id = (cur_id + 1) % sched.n; }
        if (g == -1) g = naive();
        return g;
    }
    void check_eviction(int gpu, const string& f) {                                          // :392-400
        std::vector<string> out = ev->add(gpu, f, g_repo.host[f].total, sched.level);
        for (auto& v : out) { remove_info(v, gpu); send(v, gpu, 3); }
    }
    void send_exec(const string& f, int gpu, int status) {                                   // :402-418
        if (status == 5) {
            for (int i = 0; i < sched.n; ++i) {
                if (i == gpu) { sched.status[i] = 5; running[i] = f; send(f, i, 1); }
                else send(f, i, 0);
            }
        } else {
            sched.status[gpu] = status; running[gpu] = f; send(f, gpu, 2);
        }
    }
    void send_load(const string& f, int dst, int src) {                                      // :420-427
        if (src >= 0) { demand.insert({dst, {src, f}}); ev->lock(src, f); }                 // :442-445
        check_eviction(dst, f);
        send(f, dst, 4 + 1 + src);
    }
    void unlock_src(int dst) {                                                               // :447-453
        auto it = demand.find(dst);
        if (it == demand.end()) return;
        ev->unlock(it->second.first, it->second.second);
        demand.erase(it);
    }

    void request(int type, const string& f, const string& payload) {
        if (type == 0) {                                                                     // ExecuteAfterLoad :141-162
            sched.level[f] = 1;
            if (!payload.empty()) { int lv = std::stoi(payload); if (lv >= 0 && lv <= 2) sched.level[f] = lv; }
            int g = placement();
            if (g == -1) waiting.push_back({f, true});
            else { send_exec(f, g, 5); ack(g); }
        } else if (type == 1) {                                                              // Execute :163-185
            if (!payload.empty()) {
                int g = std::stoi(payload);
                send_load(f, g, -1); send_exec(f, g, Sched::level_to_status(sched.level[f])); ack(g);
            } else {
                int d[3]; sched.decide(f, d);
                if (d[0] == -1) waiting.push_back({f, false});
                else { send_load(f, d[0], d[1]); send_exec(f, d[0], d[2]); ack(d[0]); }
            }
        } else if (type == 3) {                                                              // Unload :186-206
            if (!payload.empty()) {
                int g = std::stoi(payload);
                if (g_repo.active[f].count(g)) { ev->force(g, f); remove_info(f, g); send(f, g, 3); }
            } else {
                std::vector<int> gpus(g_repo.active[f].begin(), g_repo.active[f].end());
                for (int g : gpus) { ev->force(g, f); remove_info(f, g); send(f, g, 3); }
            }
            ack(-1);
        } else if (type == 2) {                                                              // Load :207-214
            for (int i = 0; i < sched.n; ++i) { send_load(f, i, -1); add_info(f, i); }
            ack(-1);
        }
    }
    void complete(int id) {                                                                  // :217-262
        if (sched.status[id] == 5) { add_info(running[id], id); check_eviction(id, running[id]); }
        else if (sched.status[id] > -1 && sched.status[id] < 5) add_info(running[id], id);
        unlock_src(id);
        sched.status[id] = -1;
        if (!waiting.empty()) {
            auto next = waiting.front();
            waiting.pop_front();
            if (next.second) send_exec(next.first, id, 5);
            else {
                int d[3]; sched.decide(next.first, d);
                if (d[0] != id) { send_load(next.first, id, -1); send_exec(next.first, id, Sched::level_to_status(sched.level[next.first])); }
                else { send_load(next.first, d[0], d[1]); send_exec(next.first, d[0], d[2]); }
            }
            ack(id);
        }
    }
};

int write_trace(std::vector<string>& trace, char* out, int cap) {
    string joined;
    for (size_t i = 0; i < trace.size(); ++i) { if (i) joined += "\n"; joined += trace[i]; }
    trace.clear();
    if (out && (int)joined.size() + 1 <= cap) memcpy(out, joined.c_str(), joined.size() + 1);
    return (int)joined.size() + 1;
}

}  // namespace

// ================================================================= scenario ABI
extern "C" {

const char* tso_impl_name(void) { return "cpu-restatement"; }

void tso_reset_world(void) {
    g_repo = Repo();   // host copies are leaked, as the reference never frees them
    dev_reset();
}

void* tso_create(int server_id, uint64_t budget_bytes, int, const char* block_manager, uint64_t, int) {
    Manager* m = new Manager();
    m->id = server_id;
    if (block_manager && string(block_manager) == "Fixed") m->pool.reset(new FixedPool());
    else m->pool.reset(new BuddyPool());
    m->pool->dev = server_id;
    m->pool->budget = budget_bytes + (5ull << 30);                   // memory_manager.hpp:43-44
    m->pool->init();
    g_repo.dev[server_id];                                           // init_device_info, model_repo.hpp:74-76
    return m;
}
void tso_destroy(void* h) { delete (Manager*)h; }

void tso_track_begin(void* h, const char* f) { Manager* m = (Manager*)h; m->tracking = true; m->track_func = f; g_repo.host[f]; }
void tso_track_end(void* h, const char*) { Manager* m = (Manager*)h; m->tracking = false; m->track_func.clear(); m->pool->finish_alloc(); }
uint64_t tso_malloc(void* h, const char* f, uint64_t size, int flag) { return ((Manager*)h)->do_malloc(f, size, flag != 0); }
void tso_free(void* h, const char* f, uint64_t p) { ((Manager*)h)->do_free(f, p); }
int tso_memcpy_h2d_model(void* h, const char* f, uint64_t dst, const void* payload, uint64_t size) {
    return ((Manager*)h)->upload(f, dst, payload, size);
}
void tso_sync_done(void* h, const char* f) { ((Manager*)h)->init_readiness(f, kCuda); }
int tso_mark_access(void* h, uint64_t p) { return ((Manager*)h)->mark_access(p) ? 1 : 0; }
void tso_swap_in(void* h, const char* f, int src) { ((Manager*)h)->swap_in(f, src); }
int64_t tso_wait_ready(void*, const char*) { return 0; }
int64_t tso_swap_in_timed(void* h, const char* f, int src) {
    auto t0 = std::chrono::steady_clock::now();
    ((Manager*)h)->swap_in(f, src);
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
}
void tso_evict(void* h, const char* f) { ((Manager*)h)->evict(f); }
uint64_t tso_translate(void* h, const char* f, uint64_t p) { return ((Manager*)h)->translate(f, p); }
int tso_check_alloc(void* h, const char* f) { return ((Manager*)h)->alloc_ok(f) ? 1 : 0; }
int tso_is_model_address(void*, const char* f, uint64_t p) { return g_repo.host.count(f) && g_repo.host[f].params.count(p) ? 1 : 0; }

void tso_set_model_status(const char* f, int gpu, int full) {       // model_repo.hpp:82-90
    g_repo.dev[gpu][f].status = full ? 0 : 3;
    if (full) g_repo.active[f].insert(gpu);
    else g_repo.active[f].erase(gpu);
}
uint64_t tso_total_size(const char* f) { return g_repo.host.count(f) ? g_repo.host[f].total : 0; }

int tso_pool_chunks(void* h, uint64_t* out, int cap) {
    Manager* m = (Manager*)h;
    int n = (int)m->pool->chunks.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = m->pool->chunks[i];
    return n;
}

int tso_dump_blocks(void* h, const char* f, uint64_t* out, int cap) {
    Manager* m = (Manager*)h;
    if (!g_repo.host.count(f)) return 0;
    DevModel& d = g_repo.dev[m->id][f];
    int n = 0;
    for (auto& kv : g_repo.host[f].blocks) {
        if (out && n < cap) {
            uint64_t* o = out + 6 * n;
            uint64_t b = (uint64_t)kv.first;
            o[0] = b; o[1] = kv.second.size; o[2] = kv.second.is_model; o[3] = o[4] = o[5] = 0;
            auto it = d.blocks.find(b);
            if (it != d.blocks.end()) { o[3] = it->second.in_cuda; o[4] = it->second.cuda; o[5] = it->second.in_pin; }
        }
        ++n;
    }
    return n;
}

int tso_dump_params(void* h, const char* f, uint64_t* out, int cap) {
    Manager* m = (Manager*)h;
    if (!g_repo.host.count(f)) return 0;
    HostModel& hm = g_repo.host[f];
    DevModel& d = g_repo.dev[m->id][f];
    std::vector<uint64_t> order = g_repo.access_order[f];
    std::unordered_set<uint64_t> seen(order.begin(), order.end());
    size_t n_acc = order.size();
    std::vector<uint64_t> rest;
    for (auto& kv : hm.params) if (!seen.count(kv.first)) rest.push_back(kv.first);
    std::sort(rest.begin(), rest.end());
    order.insert(order.end(), rest.begin(), rest.end());
    int n = 0;
    for (uint64_t p : order) {
        if (out && n < cap) {
            uint64_t* o = out + 7 * n;
            o[0] = p; o[1] = hm.params[p].size; o[2] = hm.data_block[p];
            auto it = d.params.find(p);
            o[3] = it == d.params.end() ? 0 : it->second.cuda;
            o[4] = (uint64_t)-1; o[5] = 0;
            auto rf = m->ready.find(f);
            if (rf != m->ready.end() && rf->second.count(p)) { o[4] = (uint64_t)rf->second[p].first; o[5] = rf->second[p].second; }
            o[6] = (size_t)n < n_acc ? 1 : 0;
        }
        ++n;
    }
    return n;
}

int tso_read_phys(void*, uint64_t addr, void* out, uint64_t size) { memcpy(out, dev_bytes(addr), size); return 0; }
int tso_read_host_store(void*, const char* f, uint64_t p, void* out, uint64_t size) {
    if (!g_repo.host.count(f) || !g_repo.host[f].params.count(p) || g_repo.host[f].params[p].size < size) return -1;
    memcpy(out, g_repo.host[f].params[p].host, size);
    return 0;
}

void* tso_evictor_create(const char* kind, int n, uint64_t budget) {
    if (kind && string(kind) == "LRU") return new LruEvictor(n, budget);
    return new IaEvictor(n, budget);
}
void tso_evictor_destroy(void* e) { delete (EvictorBase*)e; }
int tso_evictor_check_and_add(void* ev, int g, const char* f, uint64_t size, int level, char* victims, int cap) {
    EvictorBase* e = (EvictorBase*)ev;
    e->level[f] = level;
    std::vector<string> v = e->add(g, f, size, e->level);
    string joined;
    for (size_t i = 0; i < v.size(); ++i) { if (i) joined += "\n"; joined += v[i]; }
    if ((int)joined.size() + 1 > cap) return -1;
    memcpy(victims, joined.c_str(), joined.size() + 1);
    return (int)v.size();
}
void tso_evictor_force_evict(void* e, int g, const char* f) { ((EvictorBase*)e)->force(g, f); }
void tso_evictor_lock(void* e, int g, const char* f) { ((EvictorBase*)e)->lock(g, f); }
void tso_evictor_unlock(void* e, int g, const char* f) { ((EvictorBase*)e)->unlock(g, f); }

int tso_enable_peer_access(int) { return 0; }   // no devices here

// The controller's decision functions as restated above; any number of GPUs, tables as inputs.
void* tso_sched_create(int n, const char* policy, const int* pcie_pairs, const int* nvlink) {
    Sched* s = new Sched();
    s->n = n;
    s->random_policy = policy && string(policy) == "RAND";
    s->status.assign(n, -1);
    s->pcie_pairs.assign(pcie_pairs, pcie_pairs + n);
    s->nvlink.assign(n, std::vector<int>(n, 0));
    for (int i = 0; i < n; ++i) for (int j = 0; j < n; ++j) s->nvlink[i][j] = nvlink[i * n + j];
    return s;
}
void tso_sched_destroy(void* s) { delete (Sched*)s; }
void tso_sched_set_status(void* s, int gpu, int status) { ((Sched*)s)->status[gpu] = status; }
void tso_sched_set_level(void* s, const char* f, int level) { ((Sched*)s)->level[f] = level; }
void tso_sched_decide(void* s, const char* f, int* out3) { ((Sched*)s)->decide(f, out3); }

void* tso_ctrl_create(int n, uint64_t mem_limit_bytes, const char* sched_policy, const char* evict_policy,
                      const int* pcie_pairs, const int* nvlink) {
    Ctrl* c = new Ctrl();
    c->sched.n = n;
    c->sched.random_policy = sched_policy && string(sched_policy) == "RAND";
    c->sched.status.assign(n, -1);
    c->sched.pcie_pairs.assign(pcie_pairs, pcie_pairs + n);
    c->sched.nvlink.assign(n, std::vector<int>(n, 0));
    for (int i = 0; i < n; ++i) for (int j = 0; j < n; ++j) c->sched.nvlink[i][j] = nvlink[i * n + j];
    c->ev.reset((EvictorBase*)tso_evictor_create(evict_policy, n, mem_limit_bytes));
    c->running.assign(n, string());
    return c;
}
void tso_ctrl_destroy(void* c) { delete (Ctrl*)c; }
int tso_ctrl_request(void* h, int type, const char* f, const char* payload, char* trace, int cap) {
    Ctrl* c = (Ctrl*)h;
    c->request(type, f, payload ? payload : "");
    return write_trace(c->trace, trace, cap);
}
int tso_ctrl_complete(void* h, int executor, char* trace, int cap) {
    Ctrl* c = (Ctrl*)h;
    c->complete(executor);
    return write_trace(c->trace, trace, cap);
}

}  // extern "C"
