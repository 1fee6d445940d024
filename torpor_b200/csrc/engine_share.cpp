// Introspection, sharing with other processes and raw segment launches of the swap engine
// (C ABI, third part).

#include "engine_internal.hpp"

using namespace tsw;

extern "C" {

// --------------------------------------------------------------- introspection

int tsw_dump_blocks(tsw_engine* e, const char* func, int canonical, uint64_t* out, int cap) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return 0;
    auto pit = m->place.find(e->server_id);
    int n = 0;
    for (auto& kv : m->block_order) {
        if (out && n < cap) {
            const VBlock& b = m->blocks[kv.second];
            uint64_t* o = out + 6 * n;
            o[0] = canonical ? b.canon : b.vaddr;
            o[1] = b.size;
            o[2] = b.is_model;
            o[3] = o[4] = o[5] = 0;
            if (pit != m->place.end() && (size_t)kv.second < pit->second.blocks.size() && pit->second.blocks[kv.second].known) {
                const Placement::B& pb = pit->second.blocks[kv.second];
                o[3] = pb.in_cuda;
                o[4] = canonical ? pb.canon : pb.cuda;
            }
        }
        ++n;
    }
    return n;
}

static std::vector<int> dump_order(Model* m) {
    std::vector<int> order = m->access_order;
    std::vector<int> rest;
    for (size_t i = 0; i < m->params.size(); ++i)
        if (!m->params[i].accessed) rest.push_back((int)i);
    std::sort(rest.begin(), rest.end(), [m](int a, int b) { return m->params[a].vaddr < m->params[b].vaddr; });
    order.insert(order.end(), rest.begin(), rest.end());
    return order;
}

int tsw_dump_params(tsw_engine* e, const char* func, int canonical, uint64_t* out, int cap) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return 0;
    auto pit = m->place.find(e->server_id);
    std::vector<int> order = dump_order(m);
    int n = 0;
    for (int pi : order) {
        if (out && n < cap) {
            const VParam& p = m->params[pi];
            uint64_t* o = out + 7 * n;
            o[0] = canonical ? p.canon : p.vaddr;
            o[1] = p.size;
            o[2] = canonical ? m->blocks[p.block].canon : m->blocks[p.block].vaddr;
            o[3] = 0;
            o[4] = (uint64_t)-1;
            o[5] = 0;
            if (pit != m->place.end()) {
                const Placement& pl = pit->second;
                const bool known = (size_t)pi < pl.params.size() && pl.params[pi].known;
                if (known) o[3] = canonical ? pl.params[pi].canon : pl.params[pi].cuda;
                if ((size_t)pi < pl.has_row.size() && pl.has_row[pi]) {
                    o[4] = pl.flag[pi];
                    uint64_t r = pl.phys[pi];
                    if (canonical && r != 0) {
                        if (known && r == pl.params[pi].cuda) r = pl.params[pi].canon;
                        else if (r == p.vaddr) r = p.canon;
                    }
                    o[5] = r;
                }
            }
            o[6] = p.accessed ? 1 : 0;
        }
        ++n;
    }
    return n;
}

int tsw_pool_info(tsw_engine* e, uint64_t* pool_base, uint64_t* n_chunks, uint64_t* canon_base) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    if (pool_base) *pool_base = e->pool->pool_base();
    if (n_chunks) *n_chunks = e->pool->pool_chunks();
    if (canon_base) *canon_base = kCanonBase + (uint64_t)e->server_id * kCanonStride;
    return TSW_OK;
}

int tsw_canonical_address(tsw_engine* e, const char* func, uint64_t addr, uint64_t* out) {
    if (!e || !out) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    uint64_t c = e->pool->canon_inside(addr);
    if (!c && func) {
        Model* m = repo().find(func);
        if (m)
            for (auto& b : m->blocks)
                if (b.alive && addr >= b.vaddr && addr < b.vaddr + b.size) {
                    c = b.canon + (addr - b.vaddr);
                    break;
                }
    }
    *out = c ? c : addr;
    return TSW_OK;
}

int tsw_read_phys(tsw_engine* e, uint64_t addr, void* out, uint64_t size) {
    if (!e || !out) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine holds no bytes");
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemcpy(out, (void*)addr, size, cudaMemcpyDeviceToHost));
    return TSW_OK;
}

int tsw_read_host_store(tsw_engine* e, const char* func, uint64_t vptr, void* out, uint64_t size) {
    if (!e || !func || !out) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
    auto it = m->param_by_vaddr.find(vptr);
    if (it == m->param_by_vaddr.end() || m->params[it->second].size < size) return fail(TSW_ERR_NOT_FOUND, "no such parameter");
    memcpy(out, m->params[it->second].host, size);
    return TSW_OK;
}

int tsw_checksum_resident(tsw_engine* e, const char* func, uint64_t* out, int cap) {
    if (!e || !func || !out) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine holds no bytes");
    std::vector<SumDesc> descs;
    int n_rows = 0;
    const uint32_t tile = 256u * 1024;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        Model* m = repo().find(func);
        if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
        Placement& pl = placement(m, e->server_id);
        size_placement(m, pl);
        std::vector<int> order = dump_order(m);
        n_rows = (int)order.size();
        if (n_rows > cap) return fail(TSW_ERR_BUFFER, "checksum buffer too small");
        uint64_t t = 0;
        for (int row = 0; row < n_rows; ++row) {
            const int pi = order[row];
            const VParam& p = m->params[pi];
            if (!pl.params[pi].known || !pl.blocks[p.block].in_cuda || p.size == 0) continue;
            SumDesc d;
            d.addr = pl.params[pi].cuda;
            d.bytes = p.size;
            d.first_tile = (uint32_t)t;
            d.row = (uint32_t)row;
            descs.push_back(d);
            t += (p.size + tile - 1) / tile;
        }
        memset(out, 0, sizeof(uint64_t) * 2 * n_rows);
        if (descs.empty()) return n_rows;
        TSW_CUDA(cudaSetDevice(e->cfg.device));
        cudaStream_t s = (cudaStream_t)e->stream;
        TSW_CUDA(cudaStreamSynchronize(s));
        void* d_descs = nullptr;
        void* d_out = nullptr;
        TSW_CUDA(cudaMalloc(&d_descs, sizeof(SumDesc) * descs.size()));
        TSW_CUDA(cudaMalloc(&d_out, sizeof(uint64_t) * 2 * n_rows));
        TSW_CUDA(cudaMemcpyAsync(d_descs, descs.data(), sizeof(SumDesc) * descs.size(), cudaMemcpyHostToDevice, s));
        TSW_CUDA(cudaMemsetAsync(d_out, 0, sizeof(uint64_t) * 2 * n_rows, s));
        cudaError_t le = launch_checksum((const SumDesc*)d_descs, (uint32_t)descs.size(), (uint32_t)t, tile,
                                         (unsigned long long*)d_out, e->grid_ctas, s);
        if (le == cudaSuccess) le = cudaMemcpyAsync(out, d_out, sizeof(uint64_t) * 2 * n_rows, cudaMemcpyDeviceToHost, s);
        if (le == cudaSuccess) le = cudaStreamSynchronize(s);
        cudaFree(d_descs);
        cudaFree(d_out);
        if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("checksum: ") + cudaGetErrorString(le));
        e->kernel_launches++;
    }
    return n_rows;
}

// --------------------------------------------------------------- sharing with other processes

int tsw_ipc_regions(tsw_engine* e, tsw_ipc_region* out, int cap) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine has no device memory");
    Lock g2(e->mu);
    std::vector<std::pair<uint64_t, uint64_t>> regs;
    e->pool->regions(&regs);
    regs.emplace_back((uint64_t)e->dev_slab.base, e->dev_slab.size);
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    int n = 0;
    for (auto& r : regs) {
        if (out && n < cap) {
            out[n].base = r.first;
            out[n].size = r.second;
            cudaIpcMemHandle_t h;
            TSW_CUDA(cudaIpcGetMemHandle(&h, (void*)r.first));
            static_assert(sizeof(h) == sizeof(out[n].handle), "IPC handle size");
            memcpy(out[n].handle, &h, sizeof(h));
        }
        ++n;
    }
    return n;
}

int tsw_ipc_open(tsw_engine* e, const void* handle, uint64_t* mapped_base) {
    if (!e || !handle || !mapped_base) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine has no device");
    Lock g2(e->mu);
    std::string key((const char*)handle, sizeof(cudaIpcMemHandle_t));
    auto it = e->ipc_open.find(key);
    if (it != e->ipc_open.end()) {
        *mapped_base = it->second;
        return TSW_OK;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    e->ipc_open[key] = (uint64_t)p;
    *mapped_base = (uint64_t)p;
    return TSW_OK;
}

int tsw_pointer_info(tsw_engine* e, uint64_t addr, int* type, int* device, uint64_t* device_pointer, uint64_t* host_pointer) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine has no device");
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    cudaPointerAttributes at;
    cudaError_t err = cudaPointerGetAttributes(&at, (const void*)addr);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(TSW_ERR_CUDA, std::string("cudaPointerGetAttributes: ") + cudaGetErrorString(err));
    }
    if (type) *type = (int)at.type;
    if (device) *device = at.device;
    if (device_pointer) *device_pointer = (uint64_t)at.devicePointer;
    if (host_pointer) *host_pointer = (uint64_t)at.hostPointer;
    return TSW_OK;
}

int tsw_arena_info(tsw_engine* e, uint64_t* host_base, uint64_t* dev_base, uint64_t* size, uint64_t* used) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    if (host_base) *host_base = (uint64_t)e->arena.base;
    if (dev_base) *dev_base = e->arena.base ? (uint64_t)((int64_t)(uint64_t)e->arena.base + e->arena.dev_delta) : 0;
    if (size) *size = e->arena.size;
    if (used) *used = e->arena.used;
    return TSW_OK;
}

int tsw_arena_attach(tsw_engine* e, const char* shm_name, uint64_t size, uint64_t* dev_base) {
    if (!e || !shm_name || !dev_base || size == 0) return fail(TSW_ERR_INVALID, "bad arguments");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine has no device");
    Lock g2(e->mu);
    int fd = shm_open(shm_name, O_RDWR, 0600);
    if (fd < 0) return fail(TSW_ERR_NOT_FOUND, std::string("shm_open(") + shm_name + ") failed");
    void* p = map_shared_far(fd, size, e->server_id);
    close(fd);
    if (p == MAP_FAILED) return fail(TSW_ERR_INVALID, "mmap of the shared host arena failed");
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    cudaError_t err = cudaHostRegister(p, size, cudaHostRegisterPortable | cudaHostRegisterMapped);
    if (err != cudaSuccess) {
        munmap(p, size);
        return fail(TSW_ERR_CUDA, std::string("cudaHostRegister(shared arena): ") + cudaGetErrorString(err));
    }
    void* dp = nullptr;
    TSW_CUDA(cudaHostGetDevicePointer(&dp, p, 0));
    e->attached.push_back({p, size, (uint64_t)dp});
    *dev_base = (uint64_t)dp;
    return TSW_OK;
}

// Ask the driver what every address of a launch is before the kernel touches it.  Used when
// TORPOR_SWAP_VALIDATE=1: a pointer the driver does not know (a stale IPC mapping, an
// unregistered host range, an address of another process) is reported as an error instead
// of faulting the GPU.
static int validate_address(tsw_engine* e, const char* what, int index, uint64_t addr, uint64_t bytes) {
    if (bytes == 0) return TSW_OK;
    // Device-side aliases of registered host memory (where the device address differs from the
    // host address) are not reported by the driver; the engine knows the ones it made.
    if (e->arena.base) {
        const uint64_t lo = (uint64_t)((int64_t)(uint64_t)e->arena.base + e->arena.dev_delta);
        if (addr >= lo && addr + bytes <= lo + e->arena.size) return TSW_OK;
    }
    for (auto& a : e->attached)
        if (addr >= a.dev && addr + bytes <= a.dev + a.size) return TSW_OK;
    for (uint64_t probe : {addr, addr + bytes - 1}) {
        cudaPointerAttributes at;
        cudaError_t err = cudaPointerGetAttributes(&at, (const void*)probe);
        if (err != cudaSuccess) {
            cudaGetLastError();
            return fail(TSW_ERR_INVALID, std::string(what) + " " + std::to_string(index) + ": cudaPointerGetAttributes failed for " +
                                             std::to_string(probe) + ": " + cudaGetErrorString(err));
        }
        if (at.type == cudaMemoryTypeUnregistered)
            return fail(TSW_ERR_INVALID, std::string(what) + " " + std::to_string(index) + ": address " + std::to_string(probe) +
                                             " is not known to the CUDA driver in this process");
    }
    return TSW_OK;
}

static bool validation_on() {
    static const bool on = [] { const char* v = getenv("TORPOR_SWAP_VALIDATE"); return v && v[0] == '1'; }();
    return on;
}

int tsw_place_segments(tsw_engine* e, const tsw_segment* segs, int n, uint32_t tile_bytes, uint32_t tile_first,
                       uint32_t tile_stride, uint32_t tile_end, const tsw_publish* pub, int sync) {
    if (!e || (n > 0 && !segs) || n < 0) return fail(TSW_ERR_INVALID, "bad segment list");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    if (n == 0) return TSW_OK;
    if (tile_bytes == 0) tile_bytes = e->tile_host;
    if ((tile_bytes & 15u) || tile_stride == 0) return fail(TSW_ERR_INVALID, "tile size must be a multiple of 16 and stride positive");
    static_assert(sizeof(tsw_segment) == sizeof(PlaceDesc), "segment layout");
    Lock g2(e->mu);
    Plan plan;
    plan.descs.resize(n);
    memcpy(plan.descs.data(), segs, sizeof(PlaceDesc) * n);
    finish_plan(plan, tile_bytes);
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    cudaStream_t s = (cudaStream_t)e->stream;
    // launch scratch: grown on demand, reused by the next call once the stream has drained
    const uint64_t need_d = sizeof(PlaceDesc) * (uint64_t)n, need_f = sizeof(uint32_t) * ((uint64_t)n + 1);
    if (e->raw_cap < (uint64_t)n) {
        TSW_CUDA(cudaStreamSynchronize(s));
        if (e->raw_d_descs) cudaFree(e->raw_d_descs);
        if (e->raw_d_first) cudaFree(e->raw_d_first);
        if (e->raw_h) cudaFreeHost(e->raw_h);
        e->raw_d_descs = e->raw_d_first = e->raw_h = nullptr;
        e->raw_cap = 0;
        const uint64_t cap = std::max<uint64_t>((uint64_t)n, 1024);
        TSW_CUDA(cudaMalloc(&e->raw_d_descs, sizeof(PlaceDesc) * cap));
        TSW_CUDA(cudaMalloc(&e->raw_d_first, sizeof(uint32_t) * (cap + 1)));
        TSW_CUDA(cudaHostAlloc(&e->raw_h, sizeof(PlaceDesc) * cap + sizeof(uint32_t) * (cap + 1), cudaHostAllocDefault));
        e->raw_cap = cap;
    } else {
        TSW_CUDA(cudaStreamSynchronize(s));  // the staging buffer may still feed the previous launch
    }
    uint8_t* hs = (uint8_t*)e->raw_h;
    memcpy(hs, plan.descs.data(), need_d);
    memcpy(hs + sizeof(PlaceDesc) * e->raw_cap, plan.first.data(), need_f);
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_start, s));
    TSW_CUDA(cudaMemcpyAsync(e->raw_d_descs, hs, need_d, cudaMemcpyHostToDevice, s));
    TSW_CUDA(cudaMemcpyAsync(e->raw_d_first, hs + sizeof(PlaceDesc) * e->raw_cap, need_f, cudaMemcpyHostToDevice, s));
    PlaceArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = (const PlaceDesc*)e->raw_d_descs;
    a.first_tile = (const uint32_t*)e->raw_d_first;
    a.n_descs = (uint32_t)n;
    a.tile_bytes = tile_bytes;
    a.tile_lo = tile_first;
    a.tile_hi = (tile_end != 0 && tile_end < plan.first.back()) ? tile_end : plan.first.back();
    a.tile_stride = tile_stride;
    a.system_scope = 1;
    a.status = e->d_status;
    if (pub) {
        a.done_count = (uint32_t*)pub->done_count;
        a.table_phys = (uint64_t*)pub->table_phys;
        a.table_flag = (uint32_t*)pub->table_flag;
        a.host_phys = (uint64_t*)pub->host_phys;
        a.host_flag = (uint32_t*)pub->host_flag;
        a.flag_value = pub->flag_value;
        a.host_flag_value = pub->flag_value;
        a.ticket = (uint32_t*)pub->ticket;
        a.ticket_chunk = pub->ticket_chunk ? pub->ticket_chunk : 1;
        if (a.done_count && (!a.table_phys || !a.table_flag)) return fail(TSW_ERR_INVALID, "publish block needs both table columns");
    }
    if (validation_on()) {
        uint32_t max_row = 0;
        for (int i = 0; i < n; ++i) {
            // only the part of the segment whose tiles this launch can touch
            const uint64_t t0 = std::max<uint64_t>(plan.first[i], a.tile_lo), t1 = std::min<uint64_t>(plan.first[i + 1], a.tile_hi);
            if (t0 >= t1) continue;
            const uint64_t off = (t0 - plan.first[i]) * tile_bytes;
            const uint64_t end = std::min<uint64_t>((t1 - plan.first[i]) * tile_bytes, plan.descs[i].bytes);
            int rc = validate_address(e, "segment source", i, plan.descs[i].src + off, end - off);
            if (rc == TSW_OK) rc = validate_address(e, "segment destination", i, plan.descs[i].dst + off, end - off);
            if (rc != TSW_OK) return rc;
            max_row = std::max(max_row, plan.descs[i].row);
        }
        if (a.done_count) {
            int rc = validate_address(e, "tile counters", 0, (uint64_t)a.done_count, 4ull * (max_row + 1));
            if (rc == TSW_OK) rc = validate_address(e, "table column phys", 0, (uint64_t)a.table_phys, 8ull * (max_row + 1));
            if (rc == TSW_OK) rc = validate_address(e, "table column flag", 0, (uint64_t)a.table_flag, 4ull * (max_row + 1));
            if (rc != TSW_OK) return rc;
        }
    }
    const int mv = pick_mover(e, plan.descs);
    cudaError_t le = launch_place(a, mv ? e->grid_bulk : e->grid_ctas, s, mv);
    if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(le));
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_stop, s));
    e->ev_valid = true;
    if (a.tile_hi > a.tile_lo) e->kernel_launches++;
    if (a.tile_hi > a.tile_lo)
        e->bytes_moved += (uint64_t)((double)plan.bytes * (double)(a.tile_hi - a.tile_lo) / (double)plan.first.back() / tile_stride);
    if (sync) TSW_CUDA(cudaStreamSynchronize(s));
    return TSW_OK;
}

// The same tiles moved in two pipelined steps: the copy engine brings each chunk of the tile range
// from its (host) source into this GPU's memory, and the placement kernel stores the chunk to its
// destination -- another GPU's pool across NVLink, as a rule -- and counts its tiles, while the copy
// engine is already fetching the next chunk.  For a helper whose link the copy engine reads faster
// than the SMs do; the peer stores stay with the kernel, which also publishes completed rows.
int tsw_place_segments_pipelined(tsw_engine* e, const tsw_segment* segs, int n, uint32_t tile_bytes, uint32_t tile_first,
                                 uint32_t tile_end, const tsw_publish* pub, uint32_t chunk_tiles, int sync) {
    if (!e || (n > 0 && !segs) || n < 0) return fail(TSW_ERR_INVALID, "bad segment list");
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine moves no bytes");
    if (n == 0) return TSW_OK;
    if (tile_bytes == 0) tile_bytes = e->tile_dev;
    if (tile_bytes & 15u) return fail(TSW_ERR_INVALID, "tile size must be a multiple of 16");
    if (chunk_tiles == 0) chunk_tiles = std::max<uint32_t>(1u, (64u << 20) / tile_bytes);
    Lock g2(e->mu);
    Plan plan;
    plan.descs.resize(n);
    memcpy(plan.descs.data(), segs, sizeof(PlaceDesc) * n);
    finish_plan(plan, tile_bytes);
    const uint32_t lo = tile_first;
    const uint32_t hi = (tile_end != 0 && tile_end < plan.first.back()) ? tile_end : plan.first.back();
    if (hi <= lo) return TSW_OK;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    int rc = ensure_ce_stream(e);
    if (rc != TSW_OK) return rc;
    cudaStream_t s = (cudaStream_t)e->stream, s2 = (cudaStream_t)e->stream_ce;
    TSW_CUDA(cudaStreamSynchronize(s));     // scratch, staging and the previous call's kernels
    TSW_CUDA(cudaStreamSynchronize(s2));
    // this call's share, resident in this GPU's memory while it is on its way: tile t at (t - lo) * tile_bytes
    const uint64_t share = (uint64_t)(hi - lo) * tile_bytes;
    if (e->stage_cap < share) {
        if (e->stage_buf) cudaFree(e->stage_buf);
        e->stage_buf = nullptr;
        e->stage_cap = 0;
        const uint64_t cap = (share + (256ull << 20) - 1) / (256ull << 20) * (256ull << 20);
        TSW_CUDA(cudaMalloc(&e->stage_buf, cap));
        e->stage_cap = cap;
    }
    const uint64_t need_d = sizeof(PlaceDesc) * (uint64_t)n, need_f = sizeof(uint32_t) * ((uint64_t)n + 1);
    if (e->raw_cap < (uint64_t)n) {
        if (e->raw_d_descs) cudaFree(e->raw_d_descs);
        if (e->raw_d_first) cudaFree(e->raw_d_first);
        if (e->raw_h) cudaFreeHost(e->raw_h);
        e->raw_d_descs = e->raw_d_first = e->raw_h = nullptr;
        e->raw_cap = 0;
        const uint64_t cap = std::max<uint64_t>((uint64_t)n, 1024);
        TSW_CUDA(cudaMalloc(&e->raw_d_descs, sizeof(PlaceDesc) * cap));
        TSW_CUDA(cudaMalloc(&e->raw_d_first, sizeof(uint32_t) * (cap + 1)));
        TSW_CUDA(cudaHostAlloc(&e->raw_h, sizeof(PlaceDesc) * cap + sizeof(uint32_t) * (cap + 1), cudaHostAllocDefault));
        e->raw_cap = cap;
    }
    // the kernel's table: every segment reads from where its bytes will sit in the staging area
    const uint64_t stage = (uint64_t)e->stage_buf;
    std::vector<uint64_t> host_src(n);
    for (int i = 0; i < n; ++i) {
        host_src[i] = plan.descs[i].src;
        plan.descs[i].src = stage + ((uint64_t)plan.first[i] - (uint64_t)lo) * tile_bytes;   // modulo 2^64 below `lo`: never touched there
    }
    uint8_t* hs = (uint8_t*)e->raw_h;
    memcpy(hs, plan.descs.data(), need_d);
    memcpy(hs + sizeof(PlaceDesc) * e->raw_cap, plan.first.data(), need_f);
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_start, s));
    TSW_CUDA(cudaMemcpyAsync(e->raw_d_descs, hs, need_d, cudaMemcpyHostToDevice, s));
    TSW_CUDA(cudaMemcpyAsync(e->raw_d_first, hs + sizeof(PlaceDesc) * e->raw_cap, need_f, cudaMemcpyHostToDevice, s));
    PlaceArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = (const PlaceDesc*)e->raw_d_descs;
    a.first_tile = (const uint32_t*)e->raw_d_first;
    a.n_descs = (uint32_t)n;
    a.tile_bytes = tile_bytes;
    a.tile_stride = 1;
    a.system_scope = 1;
    a.status = e->d_status;
    if (pub) {
        a.done_count = (uint32_t*)pub->done_count;
        a.table_phys = (uint64_t*)pub->table_phys;
        a.table_flag = (uint32_t*)pub->table_flag;
        a.host_phys = (uint64_t*)pub->host_phys;
        a.host_flag = (uint32_t*)pub->host_flag;
        a.flag_value = pub->flag_value;
        a.host_flag_value = pub->flag_value;
        if (a.done_count && (!a.table_phys || !a.table_flag)) return fail(TSW_ERR_INVALID, "publish block needs both table columns");
    }
    int seg = 0;    // first segment that reaches into the current chunk
    for (uint32_t t0 = lo; t0 < hi; t0 += chunk_tiles) {
        const uint32_t t1 = (hi - t0 > chunk_tiles) ? t0 + chunk_tiles : hi;
        while (seg < n && plan.first[seg + 1] <= t0) ++seg;
        for (int i = seg; i < n && plan.first[i] < t1; ++i) {
            const uint64_t a0 = std::max<uint64_t>(t0, plan.first[i]), a1 = std::min<uint64_t>(t1, plan.first[i + 1]);
            if (a1 <= a0) continue;
            const uint64_t off0 = (a0 - plan.first[i]) * tile_bytes;
            const uint64_t off1 = std::min<uint64_t>((a1 - plan.first[i]) * tile_bytes, plan.descs[i].bytes);
            if (off1 <= off0) continue;
            TSW_CUDA(cudaMemcpyAsync((void*)(plan.descs[i].src + off0), (const void*)(host_src[i] + off0), off1 - off0,
                                     cudaMemcpyDefault, s2));
        }
        TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_ce, s2));
        TSW_CUDA(cudaStreamWaitEvent(s, (cudaEvent_t)e->ev_ce, 0));
        a.tile_lo = t0;
        a.tile_hi = t1;
        cudaError_t le = launch_place(a, e->grid_ctas, s, 0);
        if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(le));
        e->kernel_launches++;
    }
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_stop, s));
    e->ev_valid = true;
    e->bytes_moved += (uint64_t)((double)plan.bytes * (double)(hi - lo) / (double)plan.first.back());
    if (sync) TSW_CUDA(cudaStreamSynchronize(s));
    return TSW_OK;
}

int tsw_stats(tsw_engine* e, uint64_t* kernel_launches, uint64_t* bytes_moved, uint64_t* last_swap_device_ns) {
    if (!e) return fail(TSW_ERR_INVALID, "null argument");
    if (kernel_launches) *kernel_launches = e->kernel_launches.load();
    if (bytes_moved) *bytes_moved = e->bytes_moved.load();
    if (last_swap_device_ns) {
        *last_swap_device_ns = 0;
        if (!e->plan && e->ev_valid) {
            cudaSetDevice(e->cfg.device);
            if (cudaEventSynchronize((cudaEvent_t)e->ev_stop) == cudaSuccess) {
                float ms = 0;
                if (cudaEventElapsedTime(&ms, (cudaEvent_t)e->ev_start, (cudaEvent_t)e->ev_stop) == cudaSuccess)
                    *last_swap_device_ns = (uint64_t)(ms * 1e6);
            }
        }
    }
    return TSW_OK;
}

}  // extern "C"

