// Swap engine + C ABI, first part: process-wide state, helpers shared with engine_swap.cpp and
// engine_share.cpp, the model repository, engine set-up and tear-down, and the cold-start
// recorders.  See include/torpor_swap.h for the contract of every entry point and the reference
// method it stands for.

#include "engine_internal.hpp"

namespace tsw {

static thread_local std::string g_err;
int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
const std::string& last_error() { return g_err; }

Repo& repo() {
    static Repo r;
    return r;
}

std::mutex g_engines_mu;
std::map<int, tsw_engine*> g_engines;  // server id -> engine of this process

namespace {

class CudaMemory : public DeviceMemory {
public:
    explicit CudaMemory(int device) : device_(device) {}
    int alloc(uint64_t size, uint64_t* phys) override {
        void* p = nullptr;
        if (cudaSetDevice(device_) != cudaSuccess) return -1;
        cudaError_t e = cudaMalloc(&p, size);
        if (e != cudaSuccess) {
            fail(TSW_ERR_CUDA, std::string("cudaMalloc: ") + cudaGetErrorString(e));
            return -1;
        }
        *phys = (uint64_t)p;
        return 0;
    }
    int release(uint64_t phys) override {
        cudaSetDevice(device_);
        return cudaFree((void*)phys) == cudaSuccess ? 0 : -1;
    }
    bool plan_only() const override { return false; }
private:
    int device_;
};

class PlanMemory : public DeviceMemory {
public:
    int alloc(uint64_t, uint64_t*) override { return -1; }
    int release(uint64_t) override { return 0; }
    bool plan_only() const override { return true; }
};

}  // namespace

int64_t now_ns() {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

Placement& placement(Model* m, int server_id) { return m->place[server_id]; }

void size_placement(Model* m, Placement& pl) {
    if (pl.blocks.size() < m->blocks.size()) pl.blocks.resize(m->blocks.size());
    if (pl.params.size() < m->params.size()) pl.params.resize(m->params.size());
    if (pl.has_row.size() < m->params.size()) pl.has_row.resize(m->params.size(), false);
    if (pl.failed.size() < m->params.size()) pl.failed.resize(m->params.size(), false);
}

// Make room for one pointer-table row per parameter.
int ensure_rows(tsw_engine* e, Model* m, Placement& pl) {
    size_placement(m, pl);
    uint32_t need = (uint32_t)m->params.size();
    if (need <= pl.capacity) return TSW_OK;
    uint32_t cap = std::max<uint32_t>(need, 16);
    volatile uint32_t* flag;
    volatile uint64_t* phys;
    volatile uint32_t* gen;
    if (e->plan) {
        flag = (volatile uint32_t*)calloc(cap, sizeof(uint32_t));
        phys = (volatile uint64_t*)calloc(cap, sizeof(uint64_t));
        gen = (volatile uint32_t*)calloc(cap, sizeof(uint32_t));
        if (!flag || !phys || !gen) return fail(TSW_ERR_INVALID, "out of host memory for the pointer table");
    } else {
        flag = (volatile uint32_t*)e->host_slab.take(sizeof(uint32_t) * cap);
        phys = (volatile uint64_t*)e->host_slab.take(sizeof(uint64_t) * cap);
        gen = (volatile uint32_t*)e->host_slab.take(sizeof(uint32_t) * cap);
        void* hd = e->host_slab.take(sizeof(PlaceDesc) * cap);
        void* hf = e->host_slab.take(sizeof(uint32_t) * (cap + 1));
        void* dp = e->dev_slab.take(sizeof(uint64_t) * cap);
        void* df = e->dev_slab.take(sizeof(uint32_t) * cap);
        void* dc = e->dev_slab.take(sizeof(uint32_t) * cap);
        void* dk = e->dev_slab.take(256);
        void* dd = e->dev_slab.take(sizeof(PlaceDesc) * cap);
        void* dt = e->dev_slab.take(sizeof(uint32_t) * (cap + 1));
        if (!flag || !phys || !gen || !hd || !hf || !dp || !df || !dc || !dd || !dt || !dk)
            return fail(TSW_ERR_POOL_EXHAUSTED, "pointer-table slab exhausted");
        memset((void*)flag, 0, sizeof(uint32_t) * cap);
        memset((void*)phys, 0, sizeof(uint64_t) * cap);
        memset((void*)gen, 0, sizeof(uint32_t) * cap);
        if (pl.capacity) {
            // a model that gained parameters after its first placement: the rows published so far
            // move to the larger device table as well (the old arrays stay in the slab until a reset)
            cudaStream_t s = (cudaStream_t)e->stream;
            if (cudaSetDevice(e->cfg.device) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess ||
                cudaMemcpy(dp, pl.d_table_phys, sizeof(uint64_t) * pl.capacity, cudaMemcpyDeviceToDevice) != cudaSuccess ||
                cudaMemcpy(df, pl.d_table_flag, sizeof(uint32_t) * pl.capacity, cudaMemcpyDeviceToDevice) != cudaSuccess)
                return fail(TSW_ERR_CUDA, "moving the device pointer table to a larger one failed");
        }
        pl.h_descs = hd;
        pl.h_first = (uint32_t*)hf;
        pl.d_table_phys = (uint64_t*)dp;
        pl.d_table_flag = (uint32_t*)df;
        pl.d_done = (uint32_t*)dc;
        pl.d_ticket = (uint32_t*)dk;
        pl.d_descs = dd;
        pl.d_first = (uint32_t*)dt;
        // the device slab is zero-filled at creation, so the tile counters start at 0
    }
    for (uint32_t i = 0; i < pl.capacity; ++i) {
        flag[i] = pl.flag[i];
        phys[i] = pl.phys[i];
        gen[i] = pl.gen[i];
    }
    if (e->plan && pl.capacity) {   // freed with the placement: a waiter outside the lock may still be reading them
        pl.retired_rows.push_back((void*)pl.flag);
        pl.retired_rows.push_back((void*)pl.phys);
        pl.retired_rows.push_back((void*)pl.gen);
    }
    pl.flag = flag;
    pl.phys = phys;
    pl.gen = gen;
    pl.capacity = cap;
    return TSW_OK;
}

// The two host-visible columns are written by the placement kernel (through the host mapping)
// or by the host under the engine lock, and read by waiters without the lock: address first,
// then the flag with release order; readers take the flag with acquire order.
void set_row(Placement& pl, int idx, uint32_t flag, uint64_t phys) {
    __atomic_store_n(const_cast<uint64_t*>(&pl.phys[idx]), phys, __ATOMIC_RELAXED);
    __atomic_store_n(const_cast<uint32_t*>(&pl.flag[idx]), flag, __ATOMIC_RELEASE);
}

// init_model_readiness (memory_manager.hpp:234-238): add a row for every parameter
// that has none yet; existing rows keep their state.
int init_readiness(tsw_engine* e, Model* m, Placement& pl, uint32_t flag) {
    int rc = ensure_rows(e, m, pl);
    if (rc != TSW_OK) return rc;
    for (size_t i = 0; i < m->params.size(); ++i) {
        if (!pl.has_row[i]) {
            pl.has_row[i] = true;
            set_row(pl, (int)i, flag, m->params[i].vaddr);
        }
    }
    pl.readiness_init = true;
    return TSW_OK;
}

uint8_t* alloc_mirror(tsw_engine* e, uint64_t size) {
    if (e->plan) return (uint8_t*)malloc(size ? size : 1);
    if (e->arena.base) {
        uint64_t off = (e->arena.used + 4095) / 4096 * 4096;
        if (off + size <= e->arena.size) {
            e->arena.used = off + size;
            return e->arena.base + off;
        }
    }
    void* p = nullptr;
    cudaSetDevice(e->cfg.device);
    unsigned flags = cudaHostAllocPortable | cudaHostAllocMapped;
    if (e->host_store_mode & TSW_STORE_WRITE_COMBINED) flags |= cudaHostAllocWriteCombined;
    cudaError_t err = cudaHostAlloc(&p, size ? size : 1, flags);
    if (err != cudaSuccess) {
        fail(TSW_ERR_CUDA, std::string("cudaHostAlloc(model store): ") + cudaGetErrorString(err));
        return nullptr;
    }
    e->loose_host.push_back(p);
    return (uint8_t*)p;
}

// Device-visible address of a byte of the host store.
uint64_t host_dev_addr(tsw_engine* owner, const uint8_t* p) {
    if (owner && owner->arena.base && p >= owner->arena.base && p < owner->arena.base + owner->arena.size)
        return (uint64_t)((int64_t)(uint64_t)p + owner->arena.dev_delta);
    return (uint64_t)p;  // cudaHostAlloc'ed memory is addressed identically on host and device
}

// find_block_ephe_ptr_mapping (model_repo.hpp:111-122)
bool cache_interior_pointer(Model* m, uint64_t addr) {
    if (m->data_block.count(addr)) return true;
    for (auto& kv : m->block_order) {
        VBlock& b = m->blocks[kv.second];
        if (addr >= b.vaddr && addr < b.vaddr + b.size) {
            m->data_block[addr] = kv.second;
            b.ephe.push_back(addr);
            return true;
        }
    }
    return false;
}

// get_phy_address (memory_manager.hpp:542-568)
uint64_t phy_address(tsw_engine* e, Model* m, uint64_t ptr, bool search_amid) {
    if (!m) return ptr;
    auto it = m->data_block.find(ptr);
    if (it == m->data_block.end()) {
        // The reference's valid_memory_address caches the mapping but always answers
        // "no" (:293-298), so an interior pointer is returned untranslated the first
        // time it is seen and translated from then on.
        if (search_amid) cache_interior_pointer(m, ptr);
        return ptr;
    }
    Placement& pl = placement(m, e->server_id);
    size_placement(m, pl);
    const Placement::B& b = pl.blocks[it->second];
    if (b.in_cuda && b.cuda != 0) return ptr - m->blocks[it->second].vaddr + b.cuda;
    return ptr;
}

WaitResult wait_row(tsw_engine* e, Placement& pl, int idx, int64_t timeout_ns) {
    const int64_t deadline = now_ns() + (timeout_ns < 0 ? 0 : timeout_ns);
    int spins = 0;
    while (row_flag(pl, idx) != TSW_READY_CUDA) {
        if (e->h_status && *e->h_status)
            return {fail(TSW_ERR_KERNEL, *e->h_status == 2 ? "placement kernel gave up waiting for a bulk copy" : "placement kernel reported an inconsistent tile table"), 0};
        if ((++spins & 63) == 0) {
            if (now_ns() > deadline) return {fail(TSW_ERR_TIMEOUT, "parameter did not become ready in time"), 0};
            if (spins > 4096) std::this_thread::yield();
        }
    }
    return {TSW_OK, __atomic_load_n(const_cast<const uint64_t*>(&pl.phys[idx]), __ATOMIC_RELAXED)};
}

// Map a shared-memory arena at an address far away from where the CUDA driver keeps its own
// mappings.  A mapping that the kernel had placed next to the driver's was seen to vanish from
// the process on the first kernel launch that followed (the driver re-maps ranges it considers
// its own), which left the registered store unmapped under a running kernel.
void* map_shared_far(int fd, uint64_t size, int slot) {
    // 1 TiB apart from 32 TiB up to 95 TiB: inside the 47-bit user address space, above the heap and
    // below the stacks and libraries, and clear of the driver's zone.  Each process starts probing at
    // its own slot so that the arenas of one job do not compete for the same hint.
    const uint64_t base = 0x200000000000ull, stride = 1ull << 40;
    const int slots = 64;
    if (size <= stride) {
        for (int j = 0; j < slots; ++j) {
            const uint64_t hint = base + (uint64_t)(((slot % slots) + slots + j) % slots) * stride;
            void* p = mmap((void*)hint, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED_NOREPLACE, fd, 0);
            if (p == MAP_FAILED) continue;   // taken
            if ((uint64_t)p == hint) return p;
            munmap(p, size);                 // an old kernel ignored the flag and placed it elsewhere
        }
    }
    return mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
}

int make_arena(tsw_engine* e) {
    const uint64_t size = e->cfg.host_arena_bytes;
    if (size == 0) return TSW_OK;
    HostArena& a = e->arena;
    if (e->cfg.host_arena_shm && e->cfg.host_arena_shm[0]) {
        a.shm_name = e->cfg.host_arena_shm;
        a.shm_fd = shm_open(a.shm_name.c_str(), O_CREAT | O_RDWR, 0600);
        if (a.shm_fd < 0) return fail(TSW_ERR_INVALID, "shm_open failed for the host arena");
        if (ftruncate(a.shm_fd, (off_t)size) != 0) return fail(TSW_ERR_INVALID, "ftruncate failed for the host arena");
        void* p = map_shared_far(a.shm_fd, size, e->server_id);
        if (p == MAP_FAILED) return fail(TSW_ERR_INVALID, "mmap failed for the host arena");
        a.base = (uint8_t*)p;
        a.size = size;
        a.owner = true;
        if (e->host_store_mode & TSW_STORE_HUGE_PAGES) a.huge = madvise(p, size, MADV_HUGEPAGE) == 0;
        TSW_CUDA(cudaHostRegister(p, size, cudaHostRegisterPortable | cudaHostRegisterMapped));
        void* dp = nullptr;
        TSW_CUDA(cudaHostGetDevicePointer(&dp, p, 0));
        a.dev_delta = (int64_t)(uint64_t)dp - (int64_t)(uint64_t)p;
    } else if (e->host_store_mode & TSW_STORE_HUGE_PAGES) {
        // An anonymous mapping on 2 MiB boundaries, advised to transparent huge pages before the
        // driver pins it: fewer, larger translations for the links to walk.  Whether the kernel
        // honours the advice is up to the machine (a.huge says whether it accepted the call).
        const uint64_t two_mb = 2ull << 20;
        const uint64_t len = (size + two_mb - 1) / two_mb * two_mb;
        void* raw = mmap(nullptr, len + two_mb, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
        if (raw == MAP_FAILED) return fail(TSW_ERR_INVALID, "mmap failed for the huge-page host arena");
        const uint64_t lo = ((uint64_t)raw + two_mb - 1) / two_mb * two_mb;
        if (lo > (uint64_t)raw) munmap(raw, lo - (uint64_t)raw);
        const uint64_t tail = (uint64_t)raw + len + two_mb - (lo + len);
        if (tail) munmap((void*)(lo + len), tail);
        void* p = (void*)lo;
        a.huge = madvise(p, len, MADV_HUGEPAGE) == 0;
        a.base = (uint8_t*)p;
        a.size = len;
        a.owner = true;
        a.anon = true;
        cudaError_t err = cudaHostRegister(p, len, cudaHostRegisterPortable | cudaHostRegisterMapped);
        if (err != cudaSuccess) {
            munmap(p, len);
            a.base = nullptr;
            return fail(TSW_ERR_CUDA, std::string("cudaHostRegister(huge-page arena): ") + cudaGetErrorString(err));
        }
        void* dp = nullptr;
        TSW_CUDA(cudaHostGetDevicePointer(&dp, p, 0));
        a.dev_delta = (int64_t)(uint64_t)dp - (int64_t)(uint64_t)p;
    } else {
        void* p = nullptr;
        unsigned flags = cudaHostAllocPortable | cudaHostAllocMapped;
        if (e->host_store_mode & TSW_STORE_WRITE_COMBINED) flags |= cudaHostAllocWriteCombined;
        TSW_CUDA(cudaHostAlloc(&p, size, flags));
        a.base = (uint8_t*)p;
        a.size = size;
        a.owner = true;
        a.dev_delta = 0;
    }
    return TSW_OK;
}

tsw_engine* engine_of_block_mirror(const uint8_t* p) {
    std::lock_guard<std::mutex> g(g_engines_mu);
    for (auto& kv : g_engines) {
        HostArena& a = kv.second->arena;
        if (a.base && p >= a.base && p < a.base + a.size) return kv.second;
    }
    return nullptr;
}

// check_and_malloc_model (memory_manager.hpp:451-507): place every block that is not
// resident, in the reference's block order, and rebind the parameters inside it.
int place_blocks(tsw_engine* e, Model* m, Placement& pl) {
    struct Taken { int block; uint64_t phys; Placement::B before; };
    std::vector<Taken> taken;  // for roll-back
    for (auto& kv : m->block_order) {
        const int bi = kv.second;
        VBlock& vb = m->blocks[bi];
        Placement::B& b = pl.blocks[bi];
        if (b.known && b.in_cuda) continue;
        DevAddr a;
        if (e->pool->acquire(vb.size, false, &a) != 0) {
            // Nothing of a swap-in that does not fit stays behind: the blocks taken so far go back to
            // the pool and their table entries return to what they were (parameters of a block that is
            // not resident are never read, so their rebound addresses need no undoing).
            e->pool->finish_block_alloc();   // the chunks this attempt opened return to the heaps first
            for (auto& t : taken) {
                e->pool->evict(t.phys, m->blocks[t.block].size, false);
                pl.blocks[t.block] = t.before;
            }
            e->pool->finish_release_block();
            return fail(TSW_ERR_POOL_EXHAUSTED, "pool exhausted while placing " + m->name + ": " + e->pool->last_warning);
        }
        taken.push_back({bi, a.phys, b});
        b.known = true;
        b.in_cuda = true;
        b.cuda = a.phys;
        b.canon = a.canon;
        if (vb.is_model) {
            for (int pi : vb.params) {   // the rebind (:477-479)
                pl.params[pi].known = true;
                pl.params[pi].cuda = m->params[pi].vaddr - vb.vaddr + a.phys;
                pl.params[pi].canon = m->params[pi].vaddr - vb.vaddr + a.canon;
            }
        }
    }
    e->active_params.clear();
    for (int pi : m->access_order) e->active_params.insert(m->params[pi].vaddr);
    e->pool->finish_block_alloc();
    return TSW_OK;
}

// Peer access from this engine's GPU to `to_device`, enabled the first time a swap needs it (a
// replica source, or the target of a sharded swap this engine helps with) instead of for every
// pair of GPUs in the machine at start-up (controller.hpp:63-75): an engine opens no context on
// a GPU it never exchanges bytes with.
int ensure_peer(tsw_engine* e, int to_device) {
    if (e->plan || to_device == e->cfg.device || e->peers.count(to_device)) return TSW_OK;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    int can = 0;
    TSW_CUDA(cudaDeviceCanAccessPeer(&can, e->cfg.device, to_device));
    if (!can) return fail(TSW_ERR_CUDA, "GPU " + std::to_string(e->cfg.device) + " has no peer access to GPU " + std::to_string(to_device));
    cudaError_t pe = cudaDeviceEnablePeerAccess(to_device, 0);
    if (pe == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
    else if (pe != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(pe));
    e->peers.insert(to_device);
    return TSW_OK;
}

// The second transfer stream (copy-engine moves) and the event that joins it to the first; made on first use.
int ensure_ce_stream(tsw_engine* e) {
    if (e->stream_ce) return TSW_OK;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    cudaStream_t s2;
    cudaEvent_t ev;
    int lo_prio = 0, hi_prio = 0;
    TSW_CUDA(cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
    TSW_CUDA(cudaStreamCreateWithPriority(&s2, cudaStreamNonBlocking, hi_prio));
    TSW_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    e->stream_ce = s2;
    e->ev_ce = ev;
    return TSW_OK;
}

uint32_t pick_tile(tsw_engine* e, bool host_side) { return host_side ? e->tile_host : e->tile_dev; }

// The bulk-copy mover needs 16-byte aligned ends; anything else goes to the load/store kernel.
int pick_mover(const tsw_engine* e, const std::vector<PlaceDesc>& descs) {
    if (e->mover != 1) return 0;
    for (auto& d : descs)
        if ((d.src | d.dst) & 15ull) return 0;
    return 1;
}

// Number the tiles; where a segment does not say how many tiles complete its row, count
// them over the segments of this list and publish the first segment's destination.
void finish_plan(Plan& p, uint32_t tile) {
    p.first.assign(p.descs.size() + 1, 0);
    uint64_t t = 0;
    std::unordered_map<uint32_t, std::pair<uint32_t, uint64_t>> rows;  // row -> (tiles, first dst)
    for (size_t i = 0; i < p.descs.size(); ++i) {
        p.first[i] = (uint32_t)t;
        const uint64_t n = (p.descs[i].bytes + tile - 1) / tile;
        t += n;
        p.bytes += p.descs[i].bytes;
        auto it = rows.find(p.descs[i].row);
        if (it == rows.end()) rows[p.descs[i].row] = std::make_pair((uint32_t)n, p.descs[i].dst);
        else it->second.first += (uint32_t)n;
    }
    p.first[p.descs.size()] = (uint32_t)t;
    for (auto& d : p.descs) {
        if (d.row_tiles == 0) {
            d.row_tiles = rows[d.row].first;
            d.row_dst = rows[d.row].second;
        }
    }
}

int upload_plan(tsw_engine* e, Placement& pl, const Plan& p) {
    memcpy(pl.h_descs, p.descs.data(), sizeof(PlaceDesc) * p.descs.size());
    memcpy(pl.h_first, p.first.data(), sizeof(uint32_t) * p.first.size());
    cudaStream_t s = (cudaStream_t)e->stream;
    TSW_CUDA(cudaMemcpyAsync(pl.d_descs, pl.h_descs, sizeof(PlaceDesc) * p.descs.size(), cudaMemcpyHostToDevice, s));
    TSW_CUDA(cudaMemcpyAsync(pl.d_first, pl.h_first, sizeof(uint32_t) * p.first.size(), cudaMemcpyHostToDevice, s));
    return TSW_OK;
}

}  // namespace tsw

using namespace tsw;

// =============================================================== C ABI

extern "C" {

const char* tsw_last_error(void) { return tsw::last_error().c_str(); }
const char* tsw_version(void) { return "torpor-swap-b200 0.1 (sm_100a)"; }

void tsw_config_default(tsw_config* c) {
    if (!c) return;
    memset(c, 0, sizeof(*c));
    c->device = 0;
    c->server_id = 0;
    c->gpu_count = 1;
    c->budget_bytes = 25ull << 30;  // default_gpu_mem_limit, controller.hpp:48
    c->pool_policy = TSW_POOL_BUDDY;
}

int tsw_repo_reset(void) {
    Repo& r = repo();
    Lock g(r.mu);
    // Page-locked mirrors belong to the engine that made them; only heap mirrors
    // (plan-only engines) are released here.
    for (auto& kv : r.models) {
        for (auto& b : kv.second->blocks)
            if (b.mirror && b.mirror_heap) free(b.mirror);
        for (auto& pk : kv.second->place) {
            Placement& pl = pk.second;
            bool plan_rows = false;
            {
                std::lock_guard<std::mutex> ge(g_engines_mu);
                auto it = g_engines.find(pk.first);
                plan_rows = it == g_engines.end() || it->second->plan;
            }
            if (plan_rows && pl.capacity) {   // rows of plan-only engines are heap memory
                free((void*)pl.flag);
                free((void*)pl.phys);
                for (void* p : pl.retired_rows) free(p);
            }
        }
    }
    r.models.clear();
    r.active_devices.clear();
    // With every model gone, what the engines hold for models can be reused: pointer-table
    // rows, launch descriptors and the host store (blocks still placed in the pools stay
    // allocated there until their engine goes away).
    std::lock_guard<std::mutex> ge(g_engines_mu);
    for (auto& kv : g_engines) {
        tsw_engine* e = kv.second;
        Lock g2(e->mu);
        e->active_params.clear();
        if (e->plan) continue;
        cudaSetDevice(e->cfg.device);
        if (e->stream) cudaStreamSynchronize((cudaStream_t)e->stream);
        e->dev_slab.used = e->dev_slab_floor;
        e->host_slab.used = e->host_slab_floor;
        if (e->dev_slab.base) cudaMemset(e->dev_slab.base + e->dev_slab_floor, 0, e->dev_slab.size - e->dev_slab_floor);
        e->arena.used = 0;
        for (void* p : e->loose_host) cudaFreeHost(p);
        e->loose_host.clear();
    }
    return TSW_OK;
}

int tsw_repo_add_model_info(const char* func, int gpu) {
    if (!func) return fail(TSW_ERR_INVALID, "null argument");
    Repo& r = repo();
    Lock g(r.mu);
    Model* m = r.get_or_create(func);
    placement(m, gpu).status = TSW_MODEL_FULL;
    r.active_devices[func].insert(gpu);
    return TSW_OK;
}

int tsw_repo_remove_model_info(const char* func, int gpu) {
    if (!func) return fail(TSW_ERR_INVALID, "null argument");
    Repo& r = repo();
    Lock g(r.mu);
    Model* m = r.get_or_create(func);
    placement(m, gpu).status = TSW_MODEL_NODATA;
    r.active_devices[func].erase(gpu);
    return TSW_OK;
}

int tsw_repo_model_status(const char* func, int gpu) {
    if (!func) return fail(TSW_ERR_INVALID, "null argument");
    Repo& r = repo();
    Lock g(r.mu);
    Model* m = r.find(func);
    if (!m) return TSW_ERR_UNKNOWN_MODEL;
    auto it = m->place.find(gpu);
    if (it == m->place.end()) return TSW_ERR_NOT_FOUND;
    return it->second.status;
}

uint64_t tsw_repo_total_size(const char* func) {
    if (!func) return 0;
    Repo& r = repo();
    Lock g(r.mu);
    Model* m = r.find(func);
    return m ? m->total_size : 0;
}

int tsw_repo_active_devices(const char* func, int* gpus, int cap) {
    if (!func) return fail(TSW_ERR_INVALID, "null argument");
    Repo& r = repo();
    Lock g(r.mu);
    auto it = r.active_devices.find(func);
    if (it == r.active_devices.end()) return 0;
    int n = 0;
    for (int gdev : it->second) {
        if (n < cap && gpus) gpus[n] = gdev;
        ++n;
    }
    return n;
}

// Everything tsw_engine_create sets up; on failure the caller releases what was made so far.
static int engine_setup(const tsw_config* cfg, tsw_engine* e) {
    e->cfg = *cfg;
    e->plan = cfg->device < 0;
    e->server_id = cfg->server_id;
    if (const char* g = getenv("TORPOR_SWAP_GUARD_NAMES")) e->guard_names = g[0] == '1';
    e->tile_host = cfg->tile_bytes_host > 0 ? (uint32_t)cfg->tile_bytes_host : 64u * 1024;
    e->tile_dev = cfg->tile_bytes_device > 0 ? (uint32_t)cfg->tile_bytes_device : 512u * 1024;
    e->host_store_mode = cfg->host_store_mode;
    if (const char* hs = getenv("TORPOR_SWAP_HOST_STORE")) e->host_store_mode = atoi(hs);
    e->ticket_chunk = cfg->ticket_chunk > 0 ? (uint32_t)cfg->ticket_chunk : 1u;
    if ((e->tile_host & 15u) || (e->tile_dev & 15u)) return fail(TSW_ERR_INVALID, "tile sizes must be multiples of 16 bytes");
    if (e->plan) {
        e->mem.reset(new PlanMemory());
    } else {
        int n = 0;
        cudaError_t err = cudaGetDeviceCount(&n);
        if (err != cudaSuccess || cfg->device >= n)
            return fail(TSW_ERR_NO_DEVICE, std::string("no usable CUDA device ") + std::to_string(cfg->device) +
                                               (err != cudaSuccess ? std::string(": ") + cudaGetErrorString(err) : ""));
        TSW_CUDA(cudaSetDevice(cfg->device));
        e->mem.reset(new CudaMemory(cfg->device));
        e->grid_ctas = cfg->grid_ctas > 0 ? cfg->grid_ctas : default_grid_ctas(cfg->device);
        e->grid_host = cfg->grid_ctas_host > 0 ? cfg->grid_ctas_host : (cfg->grid_ctas > 0 ? cfg->grid_ctas : default_grid_ctas_host(cfg->device));
        if (const char* gh = getenv("TORPOR_SWAP_GRID_HOST")) {
            if (atoi(gh) > 0) e->grid_host = atoi(gh);
        }
        e->mover = cfg->mover;
        if (const char* mv = getenv("TORPOR_SWAP_MOVER")) e->mover = atoi(mv);
        e->grid_bulk = cfg->grid_ctas > 0 ? cfg->grid_ctas : default_grid_ctas(cfg->device) / 2;
        int lo = 0, hi = 0;
        TSW_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        cudaStream_t s;
        TSW_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, hi));  // memory_manager.hpp:336
        e->stream = s;
        cudaEvent_t a, b;
        TSW_CUDA(cudaEventCreate(&a));
        TSW_CUDA(cudaEventCreate(&b));
        e->ev_start = a;
        e->ev_stop = b;
        const uint64_t slab = 32ull << 20;
        void* dp = nullptr;
        TSW_CUDA(cudaMalloc(&dp, slab));
        TSW_CUDA(cudaMemset(dp, 0, slab));
        e->dev_slab.base = (uint8_t*)dp;
        e->dev_slab.size = slab;
        void* hp = nullptr;
        TSW_CUDA(cudaHostAlloc(&hp, slab, cudaHostAllocPortable | cudaHostAllocMapped));
        e->host_slab.base = (uint8_t*)hp;
        e->host_slab.size = slab;
        // the kernels' error word lives in host-mapped memory: the device writes it, waiters read it
        e->h_status = (volatile uint32_t*)e->host_slab.take(256);
        *e->h_status = 0;
        e->d_status = (uint32_t*)e->h_status;
        // Launch scratch and the first kernel launch (module load) happen here, not on the
        // first swap: both are one-time costs, and both must precede any attach of a shared arena.
        {
            const uint64_t cap = 4096;
            TSW_CUDA(cudaMalloc(&e->raw_d_descs, sizeof(PlaceDesc) * cap));
            TSW_CUDA(cudaMalloc(&e->raw_d_first, sizeof(uint32_t) * (cap + 1)));
            TSW_CUDA(cudaHostAlloc(&e->raw_h, sizeof(PlaceDesc) * cap + sizeof(uint32_t) * (cap + 1), cudaHostAllocDefault));
            e->raw_cap = cap;
            uint8_t* warm = (uint8_t*)e->dev_slab.take(512);
            PlaceDesc d;
            memset(&d, 0, sizeof(d));
            d.src = (uint64_t)warm;
            d.dst = (uint64_t)warm + 256;
            d.bytes = 16;
            d.row_tiles = 1;
            const uint32_t first[2] = {0, 1};
            TSW_CUDA(cudaMemcpy(e->raw_d_descs, &d, sizeof(d), cudaMemcpyHostToDevice));
            TSW_CUDA(cudaMemcpy(e->raw_d_first, first, sizeof(first), cudaMemcpyHostToDevice));
            PlaceArgs warm_up;
            memset(&warm_up, 0, sizeof(warm_up));
            warm_up.descs = (const PlaceDesc*)e->raw_d_descs;
            warm_up.first_tile = (const uint32_t*)e->raw_d_first;
            warm_up.n_descs = 1;
            warm_up.tile_bytes = 64;
            warm_up.tile_hi = 1;
            warm_up.tile_stride = 1;
            warm_up.status = e->d_status;
            cudaError_t le = launch_place(warm_up, 1, s);
            if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("warm-up launch: ") + cudaGetErrorString(le));
            TSW_CUDA(cudaStreamSynchronize(s));
        }
        e->dev_slab_floor = e->dev_slab.used;
        e->host_slab_floor = e->host_slab.used;
        int rc = make_arena(e);
        if (rc != TSW_OK) return rc;
    }
    const uint64_t total = cfg->budget_bytes + kHiddenBudget;  // memory_manager.hpp:43-44
    e->pool = cfg->pool_policy == TSW_POOL_FIXED ? make_fixed_pool(total, cfg->server_id, e->mem.get())
                                                 : make_buddy_pool(total, cfg->server_id, e->mem.get());
    if (e->pool->init() != 0) return fail(TSW_ERR_CUDA, "pool allocation failed: " + tsw::last_error());
    {
        std::lock_guard<std::mutex> g(g_engines_mu);
        g_engines[cfg->server_id] = e;
    }
    return TSW_OK;
}

int tsw_engine_create(const tsw_config* cfg, tsw_engine** out) {
    if (!cfg || !out) return fail(TSW_ERR_INVALID, "null argument");
    tsw_engine* e = new tsw_engine();
    const int rc = engine_setup(cfg, e);
    if (rc != TSW_OK) {
        const std::string why = tsw::last_error();
        tsw_engine_destroy(e);   // streams, slabs, pool chunks and the arena made before the failure
        return fail(rc, why);
    }
    *out = e;
    return TSW_OK;
}

int tsw_engine_destroy(tsw_engine* e) {
    if (!e) return TSW_ERR_INVALID;
    bool registered = false;
    {
        std::lock_guard<std::mutex> g(g_engines_mu);
        auto it = g_engines.find(e->server_id);
        if (it != g_engines.end() && it->second == e) {
            g_engines.erase(it);
            registered = true;
        }
    }
    if (registered) {   // (an engine whose creation failed never owned the placements of its server id)
        // rows of the pointer table live in this engine's slabs: drop its placements
        Repo& r = repo();
        Lock g(r.mu);
        for (auto& kv : r.models) {
            auto it = kv.second->place.find(e->server_id);
            if (it == kv.second->place.end()) continue;
            if (!e->plan && !it->second.waited_rows.empty())
                tsw_release_waiters(e, kv.first.c_str());   // no stream may be left waiting on a table that goes away
            if (e->plan && it->second.capacity) {
                free((void*)it->second.flag);
                free((void*)it->second.phys);
                free((void*)it->second.gen);
                for (void* p : it->second.retired_rows) free(p);
            }
            kv.second->place.erase(it);
        }
    }
    if (!e->plan) {
        cudaSetDevice(e->cfg.device);
        if (e->stream) cudaStreamSynchronize((cudaStream_t)e->stream);
        e->pool.reset();
        for (auto& kv : e->ipc_open) cudaIpcCloseMemHandle((void*)kv.second);
        for (auto& a : e->attached) {
            cudaHostUnregister(a.host);
            munmap(a.host, a.size);
        }
        if (e->raw_d_descs) cudaFree(e->raw_d_descs);
        if (e->raw_d_first) cudaFree(e->raw_d_first);
        if (e->raw_h) cudaFreeHost(e->raw_h);
        if (e->dev_slab.base) cudaFree(e->dev_slab.base);
        if (e->host_slab.base) cudaFreeHost(e->host_slab.base);
        if (e->ev_start) cudaEventDestroy((cudaEvent_t)e->ev_start);
        if (e->ev_stop) cudaEventDestroy((cudaEvent_t)e->ev_stop);
        if (e->stream_ce) {
            cudaStreamSynchronize((cudaStream_t)e->stream_ce);
            cudaStreamDestroy((cudaStream_t)e->stream_ce);
        }
        if (e->ev_ce) cudaEventDestroy((cudaEvent_t)e->ev_ce);
        if (e->stage_buf) cudaFree(e->stage_buf);
        if (e->stream) cudaStreamDestroy((cudaStream_t)e->stream);
        // The host model store outlives the engine only as long as the repository
        // refers to it; callers reset the repository before destroying engines.
        if (e->arena.base) {
            if (e->arena.shm_fd >= 0) {
                cudaHostUnregister(e->arena.base);
                munmap(e->arena.base, e->arena.size);
                close(e->arena.shm_fd);
                if (e->arena.owner) shm_unlink(e->arena.shm_name.c_str());
            } else if (e->arena.anon) {
                cudaHostUnregister(e->arena.base);
                munmap(e->arena.base, e->arena.size);
            } else {
                cudaFreeHost(e->arena.base);
            }
        }
        for (void* p : e->loose_host) cudaFreeHost(p);
    }
    delete e;
    return TSW_OK;
}

int tsw_track_begin(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    e->tracking = true;
    e->track_func = func;
    repo().get_or_create(func)->status = TSW_MODEL_INCOMPLETE;  // start_model_load
    return TSW_OK;
}

int tsw_track_end(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    if (e->tracking) repo().get_or_create(func)->status = TSW_MODEL_FULL;  // complete_model_load
    e->tracking = false;
    e->track_func.clear();
    e->pool->finish_block_alloc();
    return TSW_OK;
}

int tsw_malloc(tsw_engine* e, const char* func, uint64_t size, int load_model_flag, uint64_t* vptr) {
    if (!e || !func || !vptr) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    DevAddr a;
    if (e->pool->acquire(size, true, &a) != 0)
        return fail(TSW_ERR_POOL_EXHAUSTED, "pool exhausted in malloc: " + e->pool->last_warning);
    Model* m = repo().get_or_create(func);
    if (e->guard_names) {
        // A block is named, for good, by the first address it was given (memory_manager.hpp:88-93).  Once
        // the model has been evicted or has come back elsewhere, that address is free again, and the pool
        // can grant it to a new block of the same model: in the reference the new block then replaces the
        // old one's entry (model_repo.hpp:133-141) and the old block's parameters are lost.  With the
        // guard on, such an address is set aside and another one is asked for.
        std::vector<DevAddr> aside;
        for (;;) {
            auto clash = m->block_by_vaddr.find(a.phys);
            if (clash == m->block_by_vaddr.end() || !m->blocks[clash->second].alive) break;
            aside.push_back(a);
            if (aside.size() > 64 || e->pool->acquire(size, true, &a) != 0) {
                e->pool->finish_block_alloc();
                for (auto& h : aside) e->pool->evict(h.phys, size, false);
                e->pool->finish_release_block();
                return fail(TSW_ERR_POOL_EXHAUSTED, "no address left that does not name another block of " + m->name);
            }
        }
        if (!aside.empty()) {
            e->pool->finish_block_alloc();      // close the lists before handing the set-aside addresses back
            for (auto& h : aside) e->pool->evict(h.phys, size, false);
            e->pool->finish_release_block();
        }
    }
    // malloc_block_for_model (model_repo.hpp:133-141)
    int bi;
    auto known = m->block_by_vaddr.find(a.phys);
    if (known != m->block_by_vaddr.end()) {
        bi = known->second;
    } else {
        bi = (int)m->blocks.size();
        m->blocks.emplace_back();
        m->block_by_vaddr[a.phys] = bi;
    }
    VBlock& b = m->blocks[bi];
    b.vaddr = a.phys;
    b.canon = a.canon;
    b.size = size;
    b.is_model = load_model_flag != 0;
    b.alive = true;
    b.ephe.clear();
    if (b.is_model) {
        b.mirror = alloc_mirror(e, size);
        b.mirror_heap = e->plan;
        b.params.clear();
        if (!b.mirror) {   // no page-locked memory for the host copy: the block is given back, the model forgets it
            e->pool->finish_block_alloc();
            e->pool->evict(a.phys, size, false);
            e->pool->finish_release_block();
            b.alive = false;
            m->block_by_vaddr.erase(a.phys);
            return TSW_ERR_CUDA;
        }
    }
    m->block_order[(void*)a.canon] = bi;
    m->total_size += size;
    Placement& pl = placement(m, e->server_id);
    size_placement(m, pl);
    pl.blocks[bi].known = true;
    pl.blocks[bi].in_cuda = true;
    pl.blocks[bi].cuda = a.phys;
    pl.blocks[bi].canon = a.canon;
    *vptr = a.phys;
    return TSW_OK;
}

int tsw_free(tsw_engine* e, const char* func, uint64_t vptr) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return TSW_OK;
    auto it = m->block_by_vaddr.find(vptr);
    if (it == m->block_by_vaddr.end()) return TSW_OK;
    const int bi = it->second;
    Placement& pl = placement(m, e->server_id);
    size_placement(m, pl);
    if (!pl.blocks[bi].known) return TSW_OK;
    VBlock& b = m->blocks[bi];
    if (b.is_model) return fail(TSW_ERR_STATE, "unexpected behaviour: free model block");
    if (pl.blocks[bi].in_cuda) e->pool->evict(pl.blocks[bi].cuda, b.size, false);
    // free_block_for_model (model_repo.hpp:144-149)
    for (uint64_t p : b.ephe) m->data_block.erase(p);
    b.ephe.clear();
    b.alive = false;
    m->block_order.erase((void*)b.canon);
    m->block_by_vaddr.erase(it);
    return TSW_OK;
}

int tsw_memcpy_h2d_model(tsw_engine* e, const char* func, uint64_t dst, const void* payload, uint64_t size,
                         void* stream) {
    // A plan-only engine may be given sizes without bytes (payload null): it records the parameter.
    if (!e || !func || (!payload && size && !e->plan)) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().get_or_create(func);
    // load_model_h2d_at_start (model_repo.hpp:151-168): find the model block around dst
    int bi = -1;
    for (size_t i = 0; i < m->blocks.size(); ++i) {
        const VBlock& b = m->blocks[i];
        if (b.alive && b.is_model && dst >= b.vaddr && dst < b.vaddr + b.size) {
            bi = (int)i;
            break;
        }
    }
    if (bi < 0) return fail(TSW_ERR_NOT_FOUND, "cudaMemcpy model fails to find malloc");
    VBlock& b = m->blocks[bi];
    if (dst + size > b.vaddr + b.size) return fail(TSW_ERR_INVALID, "upload runs past the end of its block");
    uint8_t* host = b.mirror + (dst - b.vaddr);
    if (size && payload) memcpy(host, payload, size);
    int pi;
    auto pit = m->param_by_vaddr.find(dst);
    if (pit == m->param_by_vaddr.end()) {
        pi = (int)m->params.size();
        m->params.emplace_back();
        m->param_by_vaddr[dst] = pi;
        b.params.push_back(pi);
    } else {
        pi = pit->second;
        if (m->params[pi].block != bi) {
            b.params.push_back(pi);
        }
    }
    VParam& p = m->params[pi];
    p.vaddr = dst;
    p.size = size;
    p.block = bi;
    p.host = host;
    p.canon = b.canon + (dst - b.vaddr);
    m->data_block[dst] = bi;
    Placement& pl = placement(m, e->server_id);
    size_placement(m, pl);
    pl.params[pi].known = true;
    pl.params[pi].cuda = dst;  // param_virtual_to_cuda_[dst] = {nullptr, dst} (memory_manager.hpp:129)
    pl.params[pi].canon = p.canon;
    if (!e->plan && size) {
        // Upload from the page-locked copy just made, so the transfer is truly asynchronous.
        TSW_CUDA(cudaSetDevice(e->cfg.device));
        TSW_CUDA(cudaMemcpyAsync((void*)dst, host, size, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    }
    return TSW_OK;
}

int tsw_sync_done(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().get_or_create(func);
    return init_readiness(e, m, placement(m, e->server_id), TSW_READY_CUDA);
}

int tsw_mark_access(tsw_engine* e, uint64_t vptr) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    if (!e->tracking) return 1;
    Model* m = repo().get_or_create(e->track_func);
    auto it = m->param_by_vaddr.find(vptr);
    if (it == m->param_by_vaddr.end()) return 0;
    // check_add_model_access_order (model_repo.hpp:102-109)
    m->has_access_order = true;
    VParam& p = m->params[it->second];
    if (!p.accessed) {
        p.accessed = true;
        m->access_order.push_back(it->second);
    }
    return 1;
}

static int translated(tsw_engine* e, const char* func, uint64_t vptr, uint64_t* out) {
    Model* m = repo().find(func);
    *out = phy_address(e, m, vptr, true);
    return TSW_OK;
}

int tsw_memcpy_h2d(tsw_engine* e, const char* func, uint64_t dst, const void* src, uint64_t size, void* stream) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    uint64_t phys;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        translated(e, func, dst, &phys);
    }
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemcpyAsync((void*)phys, src, size, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return TSW_OK;
}

int tsw_memcpy_d2h(tsw_engine* e, const char* func, void* dst, uint64_t src, uint64_t size, void* stream) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    uint64_t phys;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        translated(e, func, src, &phys);
    }
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemcpyAsync(dst, (void*)phys, size, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return TSW_OK;
}

int tsw_memcpy_d2d(tsw_engine* e, const char* func, uint64_t dst, uint64_t src, uint64_t size, void* stream) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    uint64_t psrc = src, pdst = dst;
    int is_param = tsw_is_model_address(e, func, src);
    if (is_param == 1) {
        // memory_manager.hpp:148-152: a parameter source is recorded as accessed and waited for
        tsw_mark_access(e, src);
        int rc = tsw_translate(e, func, src, 1, 5000000000ll, &psrc);
        if (rc != TSW_OK) return rc;
    } else {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        translated(e, func, src, &psrc);
    }
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        translated(e, func, dst, &pdst);
    }
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemcpyAsync((void*)pdst, (void*)psrc, size, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return TSW_OK;
}

int tsw_memset(tsw_engine* e, const char* func, uint64_t vptr, int value, uint64_t size, void* stream) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    uint64_t phys;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        translated(e, func, vptr, &phys);
    }
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemsetAsync((void*)phys, value, size, (cudaStream_t)stream));
    return TSW_OK;
}

}  // extern "C"
