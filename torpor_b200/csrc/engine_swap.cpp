// Swap-in, swap-out and pointer translation of the swap engine (C ABI, second part).

#include "engine_internal.hpp"

using namespace tsw;

extern "C" {

// --------------------------------------------------------------- swap-in

struct Prepared {
    Model* m = nullptr;
    Placement* pl = nullptr;
    Plan plan;
    uint32_t tile = 0;
    int src_device = -1;   // device ordinal of the replica the swap reads, if any
    bool from_host = true; // the swap reads the host store (asked for, or the source replica was unhealthy)
};

// Wait for whatever still writes into this placement's blocks: the engine's own stream and
// the streams of helper engines of a sharded swap.
static int drain_placement(tsw_engine* e, Placement& pl) {
    if (e->plan || !pl.in_flight) return TSW_OK;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream));
    if (e->stream_ce) TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream_ce));   // joined into the transfer stream, unless a launch failed half way
    for (tsw_engine* h : pl.helpers) {
        TSW_CUDA(cudaSetDevice(h->cfg.device));
        TSW_CUDA(cudaStreamSynchronize((cudaStream_t)h->stream));
    }
    pl.helpers.clear();
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    pl.in_flight = false;
    return TSW_OK;
}

// Let go of every stream that waits (tsw_translate_async) for a row of this placement that has
// not arrived, and remember those rows as failed.  The generation word each of them waits for is
// host-mapped memory, and the host writes it with a plain store: no CUDA call is made, because the
// driver gives no promise that work submitted after a stream memory wait -- on whatever stream --
// is not queued behind that wait (streams share a small number of hardware queues), and a release
// that can get stuck behind the wait it ends is no release.  The released streams run on WITHOUT
// the parameter's bytes; tsw_translate and tsw_poll_ready answer TSW_ERR_KERNEL for such rows
// until the model is swapped in again or evicted, and callers check one of them after
// synchronising.  Returns the number of rows let go.
static int release_waiters(tsw_engine* e, Placement& pl) {
    std::vector<int> stuck;
    for (int row : pl.waited_rows)
        if (row >= 0 && (uint32_t)row < pl.capacity && pl.flag[row] != TSW_READY_CUDA) stuck.push_back(row);
    pl.waited_rows.clear();
    if (e->plan || stuck.empty() || !pl.gen) return 0;
    for (int row : stuck) {
        if ((size_t)row < pl.failed.size()) pl.failed[row] = true;
        __atomic_store_n(const_cast<uint32_t*>(&pl.gen[row]), pl.epoch, __ATOMIC_RELEASE);
    }
    return (int)stuck.size();
}

// A kernel of this engine reported an error status (inconsistent tile table, or a bulk copy that
// never completed): it moved nothing for the tiles concerned and published nothing.  Taken note of
// once, at the start of the next swap or eviction on the engine: rows that were on their way are
// marked failed, their waiters are let go, their tile counters are started afresh by the next
// swap, and the status word is cleared so that later swaps are not failed by an old report.
// Caller holds the repository lock and the engine lock.
static int absorb_kernel_status(tsw_engine* e) {
    if (e->plan || !e->h_status || *e->h_status == 0) return TSW_OK;
    e->last_kernel_status = *e->h_status;
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream));
    for (auto& kv : repo().models) {
        Model* m = kv.second.get();
        auto it = m->place.find(e->server_id);
        if (it == m->place.end()) continue;
        Placement& pl = it->second;
        if (!pl.in_flight && pl.waited_rows.empty()) continue;
        size_placement(m, pl);
        for (int pi : m->access_order)
            if (pl.has_row[pi] && pl.flag[pi] != TSW_READY_CUDA) pl.failed[pi] = true;
        int rc = release_waiters(e, pl);
        if (rc < 0) return rc;
        pl.counters_dirty = true;
    }
    *e->h_status = 0;
    return TSW_OK;
}

// Everything of a swap-in that precedes the data movement: source health check, block
// placement with rebind, and the list of moves in access order.  Caller holds both locks.
static int prepare_swap(tsw_engine* e, const char* func, int src_gpu, Prepared& out, bool defer = false) {
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, std::string("model ") + func + " not found in model repo");

    // sig_trans_thread (memory_manager.hpp:213-227): an unhealthy source replica falls back to the host store
    Placement* src_pl = nullptr;
    tsw_engine* src_engine = nullptr;
    if (src_gpu >= 0) {
        auto it = m->place.find(src_gpu);
        if (it != m->place.end() && it->second.status == TSW_MODEL_FULL) {
            src_pl = &it->second;
            std::lock_guard<std::mutex> g(g_engines_mu);
            auto eit = g_engines.find(src_gpu);
            if (eit != g_engines.end()) src_engine = eit->second;
        }
        if (!src_pl || (!e->plan && !src_engine)) {
            src_pl = nullptr;
            src_gpu = -1;
        }
    }

    const bool first_time_here = m->place.find(e->server_id) == m->place.end();
    Placement& pl = placement(m, e->server_id);
    if (first_time_here) pl.status = TSW_MODEL_NODATA;  // init_device_model_info (model_repo.hpp:78-80)
    size_placement(m, pl);
    int rc;
    if (!pl.readiness_init) {
        rc = init_readiness(e, m, pl, TSW_READY_HOST);
        if (rc != TSW_OK) return rc;
    } else {
        rc = ensure_rows(e, m, pl);
        if (rc != TSW_OK) return rc;
    }
    rc = absorb_kernel_status(e);
    if (rc != TSW_OK) return rc;
    rc = drain_placement(e, pl);
    if (rc != TSW_OK) return rc;
    std::fill(pl.failed.begin(), pl.failed.end(), false);
    if (pl.counters_dirty) {
        // The last swap was abandoned with parameters half moved (a participant went away): their
        // tile counters were never re-armed by a last finisher.  Start this swap from zero.
        if (!e->plan) {
            TSW_CUDA(cudaSetDevice(e->cfg.device));
            TSW_CUDA(cudaMemsetAsync(pl.d_done, 0, sizeof(uint32_t) * pl.capacity, (cudaStream_t)e->stream));
            TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream));
        }
        pl.counters_dirty = false;
        pl.remote_rows.clear();
    }
    rc = place_blocks(e, m, pl);
    if (rc != TSW_OK) {
        const std::string why = tsw::last_error();
        release_waiters(e, pl);   // nothing of this generation will be published
        return fail(rc, why);
    }
    // A new generation starts.  Waits enqueued for the old one need no release: the generation
    // word only grows and they wait for "at least", so this generation's rows satisfy them.
    pl.waited_rows.clear();

    // transfer_model (:331-438): every accessed parameter that is not on the device yet, in access order
    const bool from_host = src_gpu < 0;
    out.from_host = from_host;
    if (!from_host && src_engine && !src_engine->plan) out.src_device = src_engine->cfg.device;
    out.tile = pick_tile(e, from_host);
    for (int pi : m->access_order) {
        if (!pl.has_row[pi] || pl.flag[pi] == TSW_READY_CUDA) continue;
        const VParam& p = m->params[pi];
        const uint64_t dst = pl.params[pi].cuda;
        if ((e->plan && !defer) || p.size == 0) {
            set_row(pl, pi, TSW_READY_CUDA, dst);
            continue;
        }
        PlaceDesc d;
        d.src = from_host ? host_dev_addr(engine_of_block_mirror(p.host), p.host) : src_pl->params[pi].cuda;
        d.dst = dst;
        d.bytes = p.size;
        d.row_dst = dst;
        d.row = (uint32_t)pi;
        d.row_tiles = 0;
        out.plan.descs.push_back(d);
    }
    if (!out.plan.descs.empty()) finish_plan(out.plan, out.tile);
    out.m = m;
    out.pl = &pl;
    return TSW_OK;
}

static int swap_in_impl(tsw_engine* e, const char* func, int src_gpu, tsw_engine* const* helpers, int n_helpers) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Prepared pr;
    int rc = prepare_swap(e, func, src_gpu, pr);
    if (rc != TSW_OK) return rc;
    Placement& pl = *pr.pl;
    Plan& plan = pr.plan;
    if (e->plan || plan.descs.empty()) return TSW_OK;
    if (pr.src_device >= 0) {
        rc = ensure_peer(e, pr.src_device);   // the kernel reads the replica in the source GPU's pool
        if (rc != TSW_OK) return rc;
    }

    TSW_CUDA(cudaSetDevice(e->cfg.device));
    cudaStream_t s = (cudaStream_t)e->stream;
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_start, s));
    rc = upload_plan(e, pl, plan);
    if (rc != TSW_OK) return rc;

    PlaceArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = (const PlaceDesc*)pl.d_descs;
    a.first_tile = pl.d_first;
    a.n_descs = (uint32_t)plan.descs.size();
    a.tile_bytes = pr.tile;
    a.tile_lo = 0;
    a.tile_hi = plan.first.back();
    a.tile_stride = 1;
    a.done_count = pl.d_done;
    a.table_phys = pl.d_table_phys;
    a.table_flag = pl.d_table_flag;
    a.host_phys = (uint64_t*)pl.phys;
    a.host_flag = (uint32_t*)pl.flag;
    a.host_gen = (uint32_t*)pl.gen;
    pl.epoch += 1;
    a.flag_value = pl.epoch;
    a.host_flag_value = TSW_READY_CUDA;
    a.system_scope = (n_helpers > 0) ? 1u : 0u;
    a.status = e->d_status;

    // From here on kernels may be writing into the placement's blocks and counters.  Should a launch
    // fail half way, the placement stays marked: the next swap or eviction drains every stream that
    // was used and starts the tile counters afresh.
    pl.in_flight = true;
    pl.counters_dirty = true;
    if (n_helpers > 0) {
        // Every participating GPU works on the front of the access order at the same time:
        // by default its CTAs draw the next tile from one counter on the target, so a link
        // that is fed faster moves more tiles; with shard_static GPU r takes tiles r, r + n, ...
        const int n = n_helpers + 1;
        for (int r = 1; r < n; ++r) {
            tsw_engine* w = helpers[r - 1];
            if (!w || w->plan) return fail(TSW_ERR_INVALID, "sharded swap needs CUDA engines as helpers");
            rc = ensure_peer(w, e->cfg.device);   // a helper stores into the target's pool and reads its tables
            if (rc != TSW_OK) return rc;
        }
        TSW_CUDA(cudaSetDevice(e->cfg.device));
        TSW_CUDA(cudaMemsetAsync(pl.d_ticket, 0, sizeof(uint32_t), s));
        TSW_CUDA(cudaStreamSynchronize(s));  // descriptors and the tile dispenser must be on the target before peers read them
        a.tile_stride = (uint32_t)n;
        if (e->cfg.shard_static == 0) {
            a.ticket = pl.d_ticket;   // tiles are drawn, not dealt: faster links take more
            a.ticket_chunk = e->ticket_chunk;
        }
        for (int r = n - 1; r >= 0; --r) {
            tsw_engine* w = r == 0 ? e : helpers[r - 1];
            PlaceArgs ar = a;
            ar.tile_lo = a.ticket ? 0u : (uint32_t)r;
            TSW_CUDA(cudaSetDevice(w->cfg.device));
            if (r != 0) {
                pl.helpers.push_back(w);
                TSW_CUDA(cudaEventRecord((cudaEvent_t)w->ev_start, (cudaStream_t)w->stream));
            }
            const int mv = pick_mover(w, plan.descs);
            cudaError_t le = launch_place(ar, mv ? w->grid_bulk : w->grid_ctas, (cudaStream_t)w->stream, mv);
            if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(le));
            if (r != 0) {
                TSW_CUDA(cudaEventRecord((cudaEvent_t)w->ev_stop, (cudaStream_t)w->stream));
                w->ev_valid = true;
            }
            w->kernel_launches++;
        }
        TSW_CUDA(cudaSetDevice(e->cfg.device));
    } else if (e->mover == 2 && pr.from_host) {
        // Copy-engine-assisted swap-in from the host store.  On this platform the SMs' reads of host
        // memory reach the link in smaller requests than the copy engine's, which costs about 7 % of
        // the rate.  So the large parameters go through the copy engine, in access order, on a second
        // stream, each followed by the publish step for its row; the kernel moves the small
        // parameters (and skips the large ones) at the same time on the transfer stream.
        rc = ensure_ce_stream(e);
        if (rc != TSW_OK) return rc;
        cudaStream_t s2 = (cudaStream_t)e->stream_ce;
        TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_ce, s));       // the descriptor upload precedes the publish kernels
        TSW_CUDA(cudaStreamWaitEvent(s2, (cudaEvent_t)e->ev_ce, 0));
        a.skip_min_bytes = e->ce_min_bytes;
        bool any_small = false;
        for (size_t k = 0; k < plan.descs.size(); ++k) {
            const PlaceDesc& d = plan.descs[k];
            if (d.bytes < e->ce_min_bytes) {
                any_small = true;
                continue;
            }
            TSW_CUDA(cudaMemcpyAsync((void*)d.dst, (const void*)d.src, d.bytes, cudaMemcpyDefault, s2));
            cudaError_t pe = launch_publish_rows(a, (uint32_t)k, (uint32_t)k + 1, s2);
            if (pe != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("publish kernel launch: ") + cudaGetErrorString(pe));
            e->kernel_launches++;
        }
        if (any_small) {
            cudaError_t le = launch_place(a, e->grid_host, s, 0);
            if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(le));
            e->kernel_launches++;
        }
        TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_ce, s2));       // the transfer stream ends when both have
        TSW_CUDA(cudaStreamWaitEvent(s, (cudaEvent_t)e->ev_ce, 0));
    } else {
        const int mv = pick_mover(e, plan.descs);
        cudaError_t le = launch_place(a, mv ? e->grid_bulk : (pr.from_host ? e->grid_host : e->grid_ctas), s, mv);
        if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(le));
        e->kernel_launches++;
    }
    pl.counters_dirty = false;
    TSW_CUDA(cudaEventRecord((cudaEvent_t)e->ev_stop, s));
    e->ev_valid = true;
    e->bytes_moved += plan.bytes;
    return TSW_OK;
}

// Swap-in whose data movement is carried out by other parties (one process per GPU): this
// engine places the blocks and rebinds exactly as tsw_swap_in does, then hands out the moves.
int tsw_swap_plan(tsw_engine* e, const char* func, tsw_segment* segs, int cap, uint32_t* tile_bytes, tsw_publish* pub) {
    if (!e || !func || !tile_bytes || !pub) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Prepared pr;
    int rc = prepare_swap(e, func, -1, pr, true);
    if (rc != TSW_OK) return rc;
    Placement& pl = *pr.pl;
    const int n = (int)pr.plan.descs.size();
    if (n > cap || (n > 0 && !segs)) return fail(TSW_ERR_BUFFER, "segment buffer too small: need " + std::to_string(n));
    static_assert(sizeof(tsw_segment) == sizeof(PlaceDesc), "segment layout");
    if (n) memcpy(segs, pr.plan.descs.data(), sizeof(PlaceDesc) * n);
    *tile_bytes = pr.tile;
    memset(pub, 0, sizeof(*pub));
    pub->done_count = (uint64_t)pl.d_done;
    pub->table_phys = (uint64_t)pl.d_table_phys;
    pub->table_flag = (uint64_t)pl.d_table_flag;
    pl.epoch += 1;
    pub->flag_value = pl.epoch;       // the generation; the host-visible rows are set by tsw_swap_commit
    pub->ticket = (uint64_t)pl.d_ticket;
    pub->ticket_chunk = e->ticket_chunk;
    pl.remote_rows.clear();
    for (auto& d : pr.plan.descs) pl.remote_rows.push_back((int)d.row);
    if (n && !e->plan) {
        TSW_CUDA(cudaSetDevice(e->cfg.device));
        TSW_CUDA(cudaMemsetAsync(pl.d_ticket, 0, sizeof(uint32_t), (cudaStream_t)e->stream));
        TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream));
        e->bytes_moved += pr.plan.bytes;
    }
    return n;
}

// After every party has finished its share of a tsw_swap_plan: take the rows the kernels
// published on the device over into the host-visible table.
int tsw_swap_commit(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
    Placement& pl = placement(m, e->server_id);
    if (pl.remote_rows.empty()) return TSW_OK;
    if (e->plan) {  // nothing moved, nothing to read back: the plan is the result
        for (int row : pl.remote_rows) set_row(pl, row, TSW_READY_CUDA, pl.params[row].cuda);
        pl.remote_rows.clear();
        return TSW_OK;
    }
    std::vector<uint32_t> flag(pl.capacity);
    std::vector<uint64_t> phys(pl.capacity);
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    TSW_CUDA(cudaMemcpy(flag.data(), pl.d_table_flag, sizeof(uint32_t) * pl.capacity, cudaMemcpyDeviceToHost));
    TSW_CUDA(cudaMemcpy(phys.data(), pl.d_table_phys, sizeof(uint64_t) * pl.capacity, cudaMemcpyDeviceToHost));
    std::vector<int> missing;
    for (int row : pl.remote_rows) {
        if (flag[row] == pl.epoch) {
            set_row(pl, row, TSW_READY_CUDA, phys[row]);
            // kernels of other processes cannot reach the host-mapped generation word: streams that wait
            // for the row are let through here, now that its bytes are known to have landed
            if (pl.gen) __atomic_store_n(const_cast<uint32_t*>(&pl.gen[row]), pl.epoch, __ATOMIC_RELEASE);
        } else {
            missing.push_back(row);
        }
    }
    // Rows still on their way stay listed: the caller may commit again once the participants have
    // finished, or give up and swap the model in by itself (which starts the counters afresh).
    pl.remote_rows.swap(missing);
    if (!pl.remote_rows.empty()) {
        pl.counters_dirty = true;
        return fail(TSW_ERR_STATE, std::to_string(pl.remote_rows.size()) + " parameters were not completed by the participants");
    }
    pl.counters_dirty = false;
    return TSW_OK;
}

int tsw_swap_in(tsw_engine* e, const char* func, int src_gpu) { return swap_in_impl(e, func, src_gpu, nullptr, 0); }

int tsw_swap_in_sharded(tsw_engine* e, const char* func, tsw_engine* const* helpers, int n_helpers) {
    if (n_helpers < 0 || (n_helpers > 0 && !helpers)) return fail(TSW_ERR_INVALID, "bad helper list");
    return swap_in_impl(e, func, -1, helpers, n_helpers);
}

int tsw_wait_ready(tsw_engine* e, const char* func, int64_t timeout_ns) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Placement* pl;
    std::vector<int> order;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        Model* m = repo().find(func);
        if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
        pl = &placement(m, e->server_id);
        if (!pl->readiness_init) return fail(TSW_ERR_STATE, "model has no readiness rows on this engine");
        for (int pi : m->access_order)
            if (pl->has_row[pi]) order.push_back(pi);
    }
    const int64_t deadline = now_ns() + timeout_ns;
    // the kernel completes parameters roughly in access order: wait from the back
    for (auto it = order.rbegin(); it != order.rend(); ++it) {
        int64_t left = deadline - now_ns();
        WaitResult w = wait_row(e, *pl, *it, left > 0 ? left : 0);
        if (w.rc != TSW_OK) {
            // The bound of every stream-ordered wait on this model: when the whole-model wait gives
            // up (time-out or kernel error), the streams queued behind its rows are let go as well.
            const std::string why = tsw::last_error();
            Lock g1(repo().mu);
            Lock g2(e->mu);
            Model* m = repo().find(func);
            if (m && m->place.count(e->server_id)) release_waiters(e, placement(m, e->server_id));
            return fail(w.rc, why);
        }
    }
    return TSW_OK;
}

int tsw_release_waiters(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
    auto it = m->place.find(e->server_id);
    if (it == m->place.end()) return 0;
    size_placement(m, it->second);
    return release_waiters(e, it->second);
}

int tsw_poll_ready(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "unknown model");
    auto it = m->place.find(e->server_id);
    if (it == m->place.end() || !it->second.readiness_init) return fail(TSW_ERR_STATE, "model has no readiness rows on this engine");
    if (e->h_status && *e->h_status) return fail(TSW_ERR_KERNEL, "placement kernel reported an inconsistent tile table");
    int waiting = 0;
    for (int pi : m->access_order) {
        if ((size_t)pi < it->second.failed.size() && it->second.failed[pi])
            return fail(TSW_ERR_KERNEL, "a parameter of the model did not arrive; the streams waiting for it were let go");
        if (it->second.has_row[pi] && it->second.flag[pi] != TSW_READY_CUDA) ++waiting;
    }
    return waiting;
}

int tsw_check_alloc(tsw_engine* e, const char* func) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return 0;
    auto it = m->place.find(e->server_id);
    if (it == m->place.end()) return 0;
    Placement& pl = it->second;
    size_placement(m, pl);
    for (auto& kv : m->block_order) {
        const Placement::B& b = pl.blocks[kv.second];
        if (!b.known || !b.in_cuda) return 0;
    }
    return 1;
}

// --------------------------------------------------------------- swap-out

int tsw_evict(tsw_engine* e, const char* func, int writeback) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m) return fail(TSW_ERR_UNKNOWN_MODEL, "try to evict unrecognized model");
    auto pit = m->place.find(e->server_id);
    if (pit == m->place.end() || !pit->second.readiness_init)
        return fail(TSW_ERR_UNKNOWN_MODEL, "try to evict unrecognized model");  // memory_manager.hpp:241-244
    Placement& pl = pit->second;
    size_placement(m, pl);

    if (!e->plan) {
        int drc = absorb_kernel_status(e);
        if (drc != TSW_OK) return drc;
        drc = drain_placement(e, pl);
        if (drc != TSW_OK) return drc;
        drc = release_waiters(e, pl);   // rows that never arrived (an abandoned plan, a kernel error): nothing may wait on
        if (drc < 0) return drc;
        TSW_CUDA(cudaSetDevice(e->cfg.device));
        if (writeback) {
            // Eviction write-back: resident parameter bytes -> host store, through the same kernel.
            Plan plan;
            for (size_t pi = 0; pi < m->params.size(); ++pi) {
                if (!pl.has_row[pi] || pl.flag[pi] != TSW_READY_CUDA) continue;
                const VParam& p = m->params[pi];
                const Placement::B& b = pl.blocks[p.block];
                if (!b.in_cuda || p.size == 0) continue;
                PlaceDesc d;
                d.src = pl.params[pi].cuda;
                d.dst = host_dev_addr(engine_of_block_mirror(p.host), p.host);
                d.bytes = p.size;
                d.row_dst = d.dst;
                d.row = (uint32_t)pi;
                d.row_tiles = 0;
                plan.descs.push_back(d);
            }
            if (!plan.descs.empty()) {
                int rc = ensure_rows(e, m, pl);
                if (rc != TSW_OK) return rc;
                finish_plan(plan, e->tile_host);
                rc = upload_plan(e, pl, plan);
                if (rc != TSW_OK) return rc;
                PlaceArgs a;
                memset(&a, 0, sizeof(a));
                a.descs = (const PlaceDesc*)pl.d_descs;
                a.first_tile = pl.d_first;
                a.n_descs = (uint32_t)plan.descs.size();
                a.tile_bytes = e->tile_host;
                a.tile_lo = 0;
                a.tile_hi = plan.first.back();
                a.tile_stride = 1;
                a.system_scope = 1;
                a.status = e->d_status;
                bool kernel_has_work = true;
                if (e->mover == 2) {
                    // as on the way in: the copy engine carries the large parameters (pool -> host store),
                    // the kernel the small ones at the same time
                    rc = ensure_ce_stream(e);
                    if (rc != TSW_OK) return rc;
                    cudaStream_t s2 = (cudaStream_t)e->stream_ce;
                    a.skip_min_bytes = e->ce_min_bytes;
                    kernel_has_work = false;
                    for (const PlaceDesc& d : plan.descs) {
                        if (d.bytes < e->ce_min_bytes) {
                            kernel_has_work = true;
                            continue;
                        }
                        TSW_CUDA(cudaMemcpyAsync((void*)d.dst, (const void*)d.src, d.bytes, cudaMemcpyDefault, s2));
                    }
                }
                if (kernel_has_work) {
                    const int mv = e->mover == 2 ? 0 : pick_mover(e, plan.descs);
                    cudaError_t le = launch_place(a, mv ? e->grid_bulk : e->grid_host, (cudaStream_t)e->stream, mv);
                    if (le != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("write-back kernel launch: ") + cudaGetErrorString(le));
                    e->kernel_launches++;
                }
                e->bytes_moved += plan.bytes;
                TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream));
                if (e->mover == 2) TSW_CUDA(cudaStreamSynchronize((cudaStream_t)e->stream_ce));
            }
        }
    }

    // evict_model (:247-256): release every resident block, in the reference's block order
    for (auto& kv : m->block_order) {
        const int bi = kv.second;
        Placement::B& b = pl.blocks[bi];
        if (!b.in_cuda) continue;
        b.in_cuda = false;
        e->pool->evict(b.cuda, m->blocks[bi].size, false);
        if (m->blocks[bi].is_model) {
            for (int pi : m->blocks[bi].params)  // reset_model_readiness (:301-309)
                if (pl.has_row[pi]) set_row(pl, pi, TSW_READY_HOST, 0);
        }
    }
    e->pool->finish_release_block();
    std::fill(pl.failed.begin(), pl.failed.end(), false);
    pl.remote_rows.clear();
    return TSW_OK;
}

// --------------------------------------------------------------- translation

int tsw_translate(tsw_engine* e, const char* func, uint64_t vptr, int search_amid, int64_t timeout_ns, uint64_t* out) {
    if (!e || !func || !out) return fail(TSW_ERR_INVALID, "null argument");
    Placement* wait_pl = nullptr;
    int wait_idx = -1;
    {
        Lock g1(repo().mu);
        Lock g2(e->mu);
        Model* m = repo().find(func);
        if (!m || m->place.find(e->server_id) == m->place.end()) {
            *out = vptr;  // memory_manager.hpp:270
            return TSW_OK;
        }
        auto pit = m->param_by_vaddr.find(vptr);
        if (pit == m->param_by_vaddr.end()) {
            *out = phy_address(e, m, vptr, search_amid != 0);
            return TSW_OK;
        }
        // check_param_readiness (:527-540)
        Placement& pl = placement(m, e->server_id);
        size_placement(m, pl);
        const int pi = pit->second;
        if (!pl.readiness_init) {
            *out = vptr;
            return TSW_OK;
        }
        if ((size_t)pi < pl.failed.size() && pl.failed[pi])
            return fail(TSW_ERR_KERNEL, "the parameter did not arrive; the streams waiting for it were let go");
        if (e->active_params.count(vptr) && pl.has_row[pi]) {
            wait_pl = &pl;
            wait_idx = pi;
        } else {
            *out = pl.params[pi].cuda;
            return TSW_OK;
        }
    }
    WaitResult w = wait_row(e, *wait_pl, wait_idx, timeout_ns);
    if (w.rc != TSW_OK) return w.rc;
    *out = w.phys;
    return TSW_OK;
}

// Stream-ordered form of get_cuda_addr.  The rebound address of a parameter is known as soon
// as its block is placed; what the executor has to wait for is the bytes.  Instead of blocking
// the host (check_param_readiness, memory_manager.hpp:527-540) this returns the address at once
// and, if the parameter is still on its way, makes `stream` wait for it: a stream memory
// operation on the row's generation word (host-mapped, next to the host-visible table columns),
// which the placement kernel writes when the row's last tile has landed.  Kernels that use the parameter can then
// be enqueued behind it before the weights have arrived.  Nothing spins on the device.
int tsw_translate_async(tsw_engine* e, const char* func, uint64_t vptr, void* stream, uint64_t* out, int* waited) {
    if (!e || !func || !out) return fail(TSW_ERR_INVALID, "null argument");
    if (waited) *waited = 0;
    if (e->plan) return fail(TSW_ERR_NO_DEVICE, "plan-only engine has no streams");
    Lock g1(repo().mu);
    Lock g2(e->mu);
    Model* m = repo().find(func);
    if (!m || m->place.find(e->server_id) == m->place.end()) {
        *out = vptr;
        return TSW_OK;
    }
    auto pit = m->param_by_vaddr.find(vptr);
    if (pit == m->param_by_vaddr.end()) {
        *out = phy_address(e, m, vptr, true);
        return TSW_OK;
    }
    Placement& pl = placement(m, e->server_id);
    size_placement(m, pl);
    const int pi = pit->second;
    if (!pl.readiness_init) {
        *out = vptr;
        return TSW_OK;
    }
    *out = pl.params[pi].cuda;
    if (!(e->active_params.count(vptr) && pl.has_row[pi])) return TSW_OK;   // as check_param_readiness: not part of the last swap
    if (pl.flag[pi] == TSW_READY_CUDA) return TSW_OK;                       // already there
    if ((size_t)pi < pl.failed.size() && pl.failed[pi])
        return fail(TSW_ERR_KERNEL, "the parameter did not arrive; the streams waiting for it were let go");
    if (!pl.in_flight && pl.remote_rows.empty())
        return fail(TSW_ERR_STATE, "parameter is neither on the device nor on its way: swap the model in first");
    typedef int (*wait_fn_t)(cudaStream_t, unsigned long long, unsigned int, unsigned int);
    static wait_fn_t wait_fn = nullptr;
    if (!wait_fn) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t err = cudaGetDriverEntryPoint("cuStreamWaitValue32", &fn, cudaEnableDefault, &qres);
        if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn)
            return fail(TSW_ERR_CUDA, "stream memory operations are not available from this driver");
        wait_fn = (wait_fn_t)fn;
    }
    TSW_CUDA(cudaSetDevice(e->cfg.device));
    // the row's host-mapped generation word (page-locked, mapped, portable: its host address is its
    // device address), so that the host can end the wait with a plain store
    const int rc = wait_fn((cudaStream_t)stream, (unsigned long long)(uintptr_t)&pl.gen[pi], pl.epoch, 0x0 /* GEQ */);
    if (rc != 0) return fail(TSW_ERR_CUDA, "cuStreamWaitValue32 failed with driver error " + std::to_string(rc));
    pl.waited_rows.push_back(pi);
    if (waited) *waited = 1;
    return TSW_OK;
}

int tsw_is_model_address(tsw_engine* e, const char* func, uint64_t vptr) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Model* m = repo().find(func);
    return (m && m->param_by_vaddr.count(vptr)) ? 1 : 0;
}

int tsw_valid_memory_address(tsw_engine* e, const char* func, uint64_t vptr) {
    if (!e || !func) return fail(TSW_ERR_INVALID, "null argument");
    Lock g1(repo().mu);
    Model* m = repo().find(func);
    if (m) cache_interior_pointer(m, vptr);
    return 0;
}

}  // extern "C"
