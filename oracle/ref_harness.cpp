// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// Exposes the reference's own swap path through the scenario ABI of
// tso_abi.h.  The reference sources are NOT copied: this translation unit
// includes include/server/{memory_manager,block_manager,model_repo,evictor}.hpp
// from the read-only reference tree (see the Makefile's REF variable), with
// ref_shim/cuda_common.hpp shadowing the one header that needs protoc.
// Private members are opened in this TU only so that tables can be dumped.

#include "cuda_common.hpp"
#include "utils.hpp"
#include "safe_ptr.hpp"
#include "spdlog/spdlog.h"
#include "spdlog/sinks/null_sink.h"
#include <sstream>
#include <list>
#include <map>
#include <thread>
#include <chrono>
#include <deque>
#include <mutex>

#define private public
#define protected public
#include "model_repo.hpp"
#include "block_manager.hpp"
#include "memory_manager.hpp"
#include "evictor.hpp"
#ifdef TORPOR_REF_WITH_CONTROLLER
// controller.hpp includes "cuda_server.hpp" from its own directory, which no include path can
// override: the executor stand-in is included first and the real header's guard is pre-defined,
// so that the real file contributes nothing.  socket_helper.hpp is shadowed by include path.
#include "ref_shim_ctrl/cuda_server.hpp"
#define INCLUDE_CUDA_SERVER_HPP_
#include "controller.hpp"   // the reference's own
#endif
#ifdef TORPOR_REF_WITH_EXECUTOR
// The reference's executor (include/server/cuda_server.hpp), unmodified.  Its constructor opens a
// log file per executor (cuda_server.hpp:57-59); inside that header the call is redirected to a
// logger without a file, so that tests leave nothing behind and can make an executor twice.
namespace spdlog {
inline std::shared_ptr<logger> torpor_fileless_logger(const std::string& name, const std::string&, bool = false) {
    return std::make_shared<logger>(name, std::make_shared<sinks::null_sink_mt>());
}
}  // namespace spdlog
#define basic_logger_mt torpor_fileless_logger
#include "cuda_server.hpp"   // the reference's own; socket_helper.hpp is shadowed by ref_shim_exec/
#undef basic_logger_mt
#endif
#undef private
#undef protected

#include "tso_abi.h"

using server::manager::MemoryManager;
using server::manager::ModelRepo;
using server::manager::BuddyBasedBlockManager;

namespace {

struct Handle {
    std::unique_ptr<MemoryManager> mm;
    int server_id = 0;
    std::vector<uint64_t> chunks;  // pool chunk bases in allocation order
    bool started = false;
};

struct QuietCout {
    std::streambuf* old = nullptr;
    std::ostringstream sink;
    QuietCout() {
        if (!getenv("TORPOR_REF_VERBOSE")) old = std::cout.rdbuf(nullptr);
    }
};
QuietCout g_quiet;

logger null_logger() {
    static logger lg = std::make_shared<spdlog::logger>("torpor_ref", std::make_shared<spdlog::sinks::null_sink_mt>());
    return lg;
}

ModelRepo& repo() { return ModelRepo::getInstance(); }

}  // namespace

extern "C" {

const char* tso_impl_name(void) {
#ifdef TORPOR_REF_FAKE_CUDA
    return "reference-headers/fake-cuda";
#else
    return "reference-headers/cuda";
#endif
}

void tso_reset_world(void) {
    ModelRepo& r = repo();
    r.model_access_order_map_.clear();
    r.model_host_info_map_.clear();  // host mirrors are leaked, as the reference never frees them
    r.model_meta_data_info_map_.clear();
    r.device_model_info_map_.clear();
    r.model_active_device_map_.clear();
#ifdef TORPOR_REF_FAKE_CUDA
    torpor_ref_fake::reset_world();
#endif
}

void* tso_create(int server_id, uint64_t budget_bytes, int gpu_count, const char* block_manager,
                 uint64_t buffer_size, int io_threads) {
    if (block_manager && std::string(block_manager) == "Fixed") setenv("BLOCK_MANAGER", "Fixed", 1);
    else unsetenv("BLOCK_MANAGER");
    setenv("BUFFER_SIZE", std::to_string(buffer_size).c_str(), 1);
    setenv("IO_THREAD_NUM", std::to_string(io_threads).c_str(), 1);

    auto* h = new Handle();
    h->server_id = server_id;
    cudaCheck(cudaSetDevice(server_id));
    h->mm.reset(new MemoryManager((size_t)budget_bytes));
    h->mm->set_logger(null_logger());
    h->mm->set_server_id(server_id);
    h->mm->start_trans_thread(gpu_count);
    h->started = true;
    if (auto* b = dynamic_cast<BuddyBasedBlockManager*>(h->mm->block_manager_.get())) {
        for (void* p : b->free_block_pool_) h->chunks.push_back((uint64_t)p);
    }
    return h;
}

void tso_destroy(void* hv) {
    auto* h = (Handle*)hv;
    if (h->started) {
        h->mm->destroy_trans_thread();
    }
    // The manager object itself is leaked on purpose: the reference has no
    // teardown for its pool, and its staging threads cannot be stopped (their
    // exit test `size_ < 0` is on an unsigned field, memory_manager.hpp:314).
    h->mm.release();
    delete h;
}

void tso_track_begin(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    h->mm->set_track_model_memory(f);
}

uint64_t tso_malloc(void* hv, const char* func, uint64_t size, int load_model_flag) {
    auto* h = (Handle*)hv;
    string f(func);
    cudaSetDevice(h->server_id);
    return (uint64_t)h->mm->cudaMallocBackend((size_t)size, load_model_flag != 0, f);
}

void tso_free(void* hv, const char* func, uint64_t vptr) {
    auto* h = (Handle*)hv;
    string f(func);
    h->mm->cudaFreeBackend((void*)vptr, f);
}

int tso_memcpy_h2d_model(void* hv, const char* func, uint64_t dst, const void* payload, uint64_t size) {
    auto* h = (Handle*)hv;
    string f(func);
    string pl((const char*)payload, (size_t)size);
    h->mm->cudaMemcpyAsyncBackendHtoD((void*)dst, pl, (cudaStream_t)0, true, f);
    cudaCheck(cudaDeviceSynchronize());
    return repo().model_host_info_map_[f].model_param_info_.count((void*)dst) ? 0 : -1;
}

void tso_sync_done(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    h->mm->init_model_readiness(f);
}

int tso_mark_access(void* hv, uint64_t vptr) {
    auto* h = (Handle*)hv;
    return h->mm->try_insert_model_access((void*)vptr) ? 1 : 0;
}

void tso_track_end(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    h->mm->unset_track_model_memory(f);
}

void tso_swap_in(void* hv, const char* func, int src_gpu) {
    auto* h = (Handle*)hv;
    string f(func);
    cudaSetDevice(h->server_id);
    h->mm->sig_trans_thread(f, src_gpu);
}

static int64_t wait_last_param(Handle* h, string& f) {
    auto t0 = std::chrono::steady_clock::now();
    auto& order = repo().model_access_order_map_[f];
    if (!order.empty()) h->mm->get_cuda_addr(f, order.back());
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
}

static void wait_staging_recycled(Handle* h, string& f) {
    // memory_manager.hpp:414-423 runs on the transfer thread after the last
    // readiness publish; an evict issued before it finishes would read in_pin_.
    auto& blocks = repo().device_model_info_map_[h->server_id][f].block_virtual_to_cuda_;
    for (int spin = 0; spin < 200000; ++spin) {
        bool any = false;
        for (auto& kv : blocks) any = any || kv.second.in_pin_;
        if (!any) return;
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int64_t tso_wait_ready(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    int64_t us = wait_last_param(h, f);
    wait_staging_recycled(h, f);
    return us;
}

int64_t tso_swap_in_timed(void* hv, const char* func, int src_gpu) {
    auto* h = (Handle*)hv;
    string f(func);
    cudaSetDevice(h->server_id);
    auto t0 = std::chrono::steady_clock::now();
    h->mm->sig_trans_thread(f, src_gpu);
    wait_last_param(h, f);
    int64_t us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    wait_staging_recycled(h, f);
    return us;
}

// The host-side pack alone: every accessed parameter copied from the pageable model store into
// the pinned mirror of its pool block by the reference's own I/O threads (pinned_io_thread,
// memory_manager.hpp:311-329; addresses from :481-483), timed from the first enqueue to the last
// completion token.  Nothing crosses to the GPU.  The model must be evicted on entry and is
// evicted again on return, with its pinned mirrors back on the free list (:414-423).
int64_t tso_pack_timed(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    cudaSetDevice(h->server_id);
    h->mm->check_and_malloc_model(f, true);
    auto& dev = repo().device_model_info_map_[h->server_id][f];
    auto& host = repo().model_host_info_map_[f];
    int count = 0;
    auto t0 = std::chrono::steady_clock::now();
    for (auto& ptr : repo().model_access_order_map_[f]) {
        h->mm->io_queue_->enqueue({f, ptr, dev.param_virtual_to_cuda_[ptr].pinned_addr_, host.model_param_info_[ptr].host_addr_,
                                   host.model_param_info_[ptr].size_});
        ++count;
    }
    // wait as the transfer thread does (:380-383): per parameter, on its readiness, taking completion
    // tokens while it is not packed yet (tokens left over from earlier swaps are never cleared, :412)
    for (auto& ptr : repo().model_access_order_map_[f])
        while (h->mm->model_param_readiness_[f]->at(ptr).first < server::manager::ParamReadiness_Pinned) h->mm->sync_io_queue_->dequeue();
    int64_t us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    for (auto& info : host.model_block_info_) {
        auto& b = dev.block_virtual_to_cuda_[info.first];
        if (b.in_pin_) {
            h->mm->free_pinend_memory(b.pinned_addr_, host.virtual_blocks_[info.first].size_);
            b.in_pin_ = false;
        }
    }
    h->mm->evict_model(f);
    return us;
}

void tso_evict(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    h->mm->evict_model(f);
}

uint64_t tso_translate(void* hv, const char* func, uint64_t vptr) {
    auto* h = (Handle*)hv;
    string f(func);
    return (uint64_t)h->mm->get_cuda_addr(f, (void*)vptr);
}

int tso_check_alloc(void* hv, const char* func) {
    auto* h = (Handle*)hv;
    string f(func);
    return h->mm->check_model_alloc_status(f) ? 1 : 0;
}

int tso_is_model_address(void* hv, const char* func, uint64_t vptr) {
    auto* h = (Handle*)hv;
    string f(func);
    return h->mm->is_model_address(f, (void*)vptr) ? 1 : 0;
}

void tso_set_model_status(const char* func, int gpu, int full) {
    string f(func);
    if (full) repo().add_model_info(f, gpu);
    else repo().remove_model_info(f, gpu);
}

uint64_t tso_total_size(const char* func) {
    string f(func);
    return repo().model_host_info_map_[f].total_size_;
}

int tso_pool_chunks(void* hv, uint64_t* out, int cap) {
    auto* h = (Handle*)hv;
    int n = (int)h->chunks.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = h->chunks[i];
    return n;
}

int tso_dump_blocks(void* hv, const char* func, uint64_t* out, int cap) {
    auto* h = (Handle*)hv;
    string f(func);
    auto& host = repo().model_host_info_map_[f];
    auto& dev = repo().device_model_info_map_[h->server_id][f];
    int n = 0;
    for (auto& kv : host.virtual_blocks_) {
        if (n < cap) {
            uint64_t* o = out + 6 * n;
            o[0] = (uint64_t)kv.first;
            o[1] = kv.second.size_;
            o[2] = kv.second.is_model_;
            auto it = dev.block_virtual_to_cuda_.find(kv.first);
            if (it == dev.block_virtual_to_cuda_.end()) { o[3] = 0; o[4] = 0; o[5] = 0; }
            else { o[3] = it->second.in_cuda_; o[4] = (uint64_t)it->second.cuda_addr_; o[5] = it->second.in_pin_; }
        }
        ++n;
    }
    return n;
}

int tso_dump_params(void* hv, const char* func, uint64_t* out, int cap) {
    auto* h = (Handle*)hv;
    string f(func);
    auto& host = repo().model_host_info_map_[f];
    auto& dev = repo().device_model_info_map_[h->server_id][f];
    std::vector<void*> order = repo().model_access_order_map_[f];
    std::unordered_set<void*> accessed(order.begin(), order.end());
    std::vector<void*> rest;
    for (auto& kv : host.model_param_info_) if (!accessed.count(kv.first)) rest.push_back(kv.first);
    std::sort(rest.begin(), rest.end(), [](void* a, void* b) { return (uint64_t)a < (uint64_t)b; });
    size_t n_acc = order.size();
    order.insert(order.end(), rest.begin(), rest.end());
    int n = 0;
    for (void* p : order) {
        if (n < cap) {
            uint64_t* o = out + 7 * n;
            o[0] = (uint64_t)p;
            o[1] = host.model_param_info_[p].size_;
            o[2] = (uint64_t)host.virtual_data_block_mapping_[p];
            auto it = dev.param_virtual_to_cuda_.find(p);
            o[3] = it == dev.param_virtual_to_cuda_.end() ? 0 : (uint64_t)it->second.cuda_addr_;
            o[4] = (uint64_t)-1; o[5] = 0;
            auto rit = h->mm->model_param_readiness_.find(f);
            if (rit != h->mm->model_param_readiness_.end() && rit->second->find(p) != rit->second->end()) {
                auto pr = rit->second->at(p);
                o[4] = (uint64_t)pr.first;
                o[5] = (uint64_t)pr.second;
            }
            o[6] = (size_t)n < n_acc ? 1 : 0;
        }
        ++n;
    }
    return n;
}

int tso_read_phys(void* hv, uint64_t addr, void* out, uint64_t size) {
    auto* h = (Handle*)hv;
    cudaSetDevice(h->server_id);
    return (int)cudaMemcpy(out, (void*)addr, (size_t)size, cudaMemcpyDeviceToHost);
}

int tso_read_host_store(void* hv, const char* func, uint64_t vptr, void* out, uint64_t size) {
    (void)hv;
    string f(func);
    auto& host = repo().model_host_info_map_[f];
    auto it = host.model_param_info_.find((void*)vptr);
    if (it == host.model_param_info_.end() || it->second.size_ < size) return -1;
    memcpy(out, it->second.host_addr_, (size_t)size);
    return 0;
}

// ---------------------------------------------------------------- evictor

struct EvictorHandle {
    std::shared_ptr<server::Evictor> ev;
    map<string, int> levels;
};

void* tso_evictor_create(const char* kind, int gpu_count, uint64_t budget) {
    auto* e = new EvictorHandle();
    if (kind && std::string(kind) == "LRU") e->ev = std::make_shared<server::LRUEvictor>(gpu_count, (size_t)budget);
    else e->ev = std::make_shared<server::InterferenceAwareEvictor>(gpu_count, (size_t)budget);
    return e;
}

void tso_evictor_destroy(void* ev) { delete (EvictorHandle*)ev; }

int tso_evictor_check_and_add(void* ev, int gpu, const char* func, uint64_t size, int level, char* victims, int cap) {
    auto* e = (EvictorHandle*)ev;
    string f(func);
    e->levels[f] = level;
    auto v = e->ev->check_and_add(gpu, f, (size_t)size, e->levels);
    std::string joined;
    for (size_t i = 0; i < v.size(); ++i) { if (i) joined += "\n"; joined += v[i]; }
    if ((int)joined.size() + 1 > cap) return -1;
    memcpy(victims, joined.c_str(), joined.size() + 1);
    return (int)v.size();
}

void tso_evictor_force_evict(void* ev, int gpu, const char* func) { string f(func); ((EvictorHandle*)ev)->ev->force_evict(gpu, f); }
void tso_evictor_lock(void* ev, int gpu, const char* func) { string f(func); ((EvictorHandle*)ev)->ev->lock(gpu, f); }
void tso_evictor_unlock(void* ev, int gpu, const char* func) { string f(func); ((EvictorHandle*)ev)->ev->unlock(gpu, f); }

// All-pairs peer access, which the reference's controller switches on at start-up for the process
// that holds every manager (controller.hpp:63-75); without it a peer copy is staged through the host.
int tso_enable_peer_access(int gpu_count) {
#ifdef TORPOR_REF_FAKE_CUDA
    (void)gpu_count;
    return 0;
#else
    int enabled = 0;
    for (int i = 0; i < gpu_count; ++i) {
        cudaSetDevice(i);
        for (int j = 0; j < gpu_count; ++j) {
            if (i == j) continue;
            int able = 0;
            cudaDeviceCanAccessPeer(&able, i, j);
            if (able) {
                cudaError_t err = cudaDeviceEnablePeerAccess(j, 0);
                if (err == cudaSuccess || err == cudaErrorPeerAccessAlreadyEnabled) ++enabled;
                cudaGetLastError();
            }
        }
    }
    return enabled;
#endif
}

// ---------------------------------------------------------------- controller decisions
#ifdef TORPOR_REF_WITH_CONTROLLER
// The reference's Controller object itself (include/server/controller.hpp), built on a 4-GPU
// stand-in: its scheduling functions (:296-389) and its load request (:420-427, with the
// eviction check :392-400 and the source pin :437-447) run unmodified; sockets are no-ops and
// executors only record the signals they are sent.
struct CtrlHandle {
    zmq::context_t ctx;
    std::unique_ptr<server::Controller> c;
};

void* tso_sched_create(int n, const char* policy, const int* pcie_pairs, const int* nvlink) {
    if (n != 4) return nullptr;   // the reference's tables are hard-coded for 4 GPUs (:116-118)
    for (int i = 0; i < 4; ++i) {
        if (pcie_pairs[i] != (int[]){1, 0, 3, 2}[i]) return nullptr;
    }
    (void)nvlink;
    torpor_ref_fake::device_count() = n;
    if (policy && std::string(policy) == "RAND") setenv("SCHEDULE_POLICY", "RAND", 1);
    else unsetenv("SCHEDULE_POLICY");
    setenv("EVICT_POLICY", "LRU", 1);
    auto* h = new CtrlHandle();
    h->c.reset(new server::Controller(null_logger(), &h->ctx));
    return h;
}
void tso_sched_destroy(void* s) { delete (CtrlHandle*)s; }
void tso_sched_set_status(void* s, int gpu, int status) { ((CtrlHandle*)s)->c->executor_status_[gpu].status_ = status; }
void tso_sched_set_level(void* s, const char* func, int level) { ((CtrlHandle*)s)->c->model_level_map_[func] = level; }
void tso_sched_decide(void* s, const char* func, int* out3) {
    string f(func);
    auto d = ((CtrlHandle*)s)->c->schedule_func_(f);
    out3[0] = d.gpu_idx_; out3[1] = d.src_swap_gpu_; out3[2] = d.status_;
}

// The controller's own loop (Controller::start, :125-264), run for exactly one event: the
// socket stand-in hands the loop one scripted request -- or puts one executor id on
// controller_sync_queue, as CUDAExecutor does when it finishes (cuda_server.hpp:298) -- and
// throws out of the endless loop at the next poll.  The executor threads start() spawns are
// joined here (the stand-in's executor returns at once).
void* tso_ctrl_create(int n, uint64_t mem_limit_bytes, const char* sched_policy, const char* evict_policy,
                      const int* pcie_pairs, const int* nvlink) {
    const uint64_t GiB = 1ull << 30;
    if (mem_limit_bytes % GiB != 0 || mem_limit_bytes / GiB < 1 || mem_limit_bytes / GiB > 24) return nullptr;
    setenv("MEM_LIMIT_IN_GB", std::to_string(mem_limit_bytes / GiB).c_str(), 1);
    void* h = tso_sched_create(n, sched_policy, pcie_pairs, nvlink);
    if (!h) return nullptr;
    // tso_sched_create built the controller with EVICT_POLICY=LRU; rebuild it if the other policy is asked for
    if (!(evict_policy && std::string(evict_policy) == "LRU")) {
        delete (CtrlHandle*)h;
        unsetenv("EVICT_POLICY");
        auto* fresh = new CtrlHandle();
        fresh->c.reset(new server::Controller(null_logger(), &fresh->ctx));
        h = fresh;
    }
    unsetenv("MEM_LIMIT_IN_GB");
    return h;
}
void tso_ctrl_destroy(void* c) { delete (CtrlHandle*)c; }

static int run_one_event(CtrlHandle* h, const std::string* request, int executor, char* out, int cap) {
    auto& st = torpor_ref_script::state();
    st.trace.clear();
    int polls = 0;
    st.next = [&](string* r) -> bool {
        if (polls++ > 0) throw torpor_ref_script::Stop();
        if (request) { *r = *request; return true; }
        server::controller_sync_queue->push(executor);
        return false;
    };
    try {
        h->c->start();
    } catch (const torpor_ref_script::Stop&) {
    }
    st.next = nullptr;
    for (auto& t : h->c->thread_vec_) if (t.joinable()) t.join();
    h->c->thread_vec_.clear();
    std::string joined;
    for (size_t i = 0; i < st.trace.size(); ++i) { if (i) joined += "\n"; joined += st.trace[i]; }
    st.trace.clear();
    if (out && (int)joined.size() + 1 <= cap) memcpy(out, joined.c_str(), joined.size() + 1);
    return (int)joined.size() + 1;
}
int tso_ctrl_request(void* c, int type, const char* func, const char* payload, char* trace, int cap) {
    const std::string req = std::to_string(type) + " " + func + " " + (payload ? payload : "");
    return run_one_event((CtrlHandle*)c, &req, -1, trace, cap);
}
int tso_ctrl_complete(void* c, int executor, char* trace, int cap) {
    return run_one_event((CtrlHandle*)c, nullptr, executor, trace, cap);
}
#endif

// ---------------------------------------------------------------- executor
#ifdef TORPOR_REF_WITH_EXECUTOR
}  // extern "C"

// src/server/kernel_lookup.cpp fills this table from the CUDA fat binaries the server links; here
// the harness registers kernel names (tso_exec_register_kernel).
map<string, const void*>& lookup() {
    static map<string, const void*> table;
    return table;
}
map<string, KernelAccessLoc>& kernel_model_access_loc() {
    static map<string, KernelAccessLoc> table;
    return table;
}

namespace {
struct Launch {
    std::string kernel;
    std::vector<std::string> args;
};
std::mutex g_launch_mu;
std::deque<std::vector<size_t>> g_expected_arg_sizes;   // byte length of every argument of the launches to come
std::vector<Launch> g_launches;

struct ExecHandle {
    zmq::context_t ctx;
    server::CUDAExecutor* ex = nullptr;   // never destroyed: the manager inside it cannot be torn down (see tso_destroy)
    std::thread loop;
    Handle view;                          // the executor's own manager, for the table dumps (not owned)
    torpor_ref_exec::Channel* channel = nullptr;
};
}  // namespace

namespace torpor_ref_fake {
void record_launch(const void* func, void** args) {
    std::lock_guard<std::mutex> g(g_launch_mu);
    Launch l;
    for (auto& kv : lookup()) if (kv.second == func) l.kernel = kv.first;
    if (!g_expected_arg_sizes.empty()) {
        std::vector<size_t> sizes = g_expected_arg_sizes.front();
        g_expected_arg_sizes.pop_front();
        for (size_t i = 0; i < sizes.size(); ++i) l.args.emplace_back((const char*)args[i], sizes[i]);
    }
    g_launches.push_back(l);
}
}  // namespace torpor_ref_fake

extern "C" {

void tso_exec_register_kernel(const char* name) {
    static char anchors[4096];
    auto& t = lookup();
    if (!t.count(name) && t.size() < sizeof(anchors)) t[name] = &anchors[t.size()];
}

void* tso_exec_create(int id, uint64_t budget_bytes, int gpu_count) {
    torpor_ref_fake::device_count() = gpu_count;
    setenv("IO_THREAD_NUM", "2", 1);            // BLOCK_MANAGER is the caller's to set, as for the server itself
    auto* h = new ExecHandle();
    h->ex = new server::CUDAExecutor(id, (size_t)budget_bytes, &h->ctx);
    h->channel = &torpor_ref_exec::channel_of((void*)&h->ex->srv_pull_handler_);
    server::CUDAExecutor* ex = h->ex;
    h->loop = std::thread([ex] {
        try {
            ex->start();
        } catch (const torpor_ref_exec::Stop&) {
        }
    });
    {   // until the loop has set itself up (pool, streams) and polls for the first time
        std::unique_lock<std::mutex> lk(h->channel->mu);
        h->channel->cv.wait(lk, [&] { return h->channel->polls > 0; });
    }
    h->view.mm.reset(&h->ex->mem_manager_);
    h->view.server_id = id;
    h->view.started = false;
    return h;
}

void* tso_exec_manager(void* hv) { return &((ExecHandle*)hv)->view; }

void tso_exec_destroy(void* hv) {
    auto* h = (ExecHandle*)hv;
    {
        std::lock_guard<std::mutex> g(h->channel->mu);
        h->channel->stop = true;
        h->channel->cv.notify_all();
    }
    if (h->loop.joinable()) h->loop.join();
    {
        std::lock_guard<std::mutex> g(h->channel->mu);
        h->channel->stop = false;
        h->channel->polls = 0;
        h->channel->inbox.clear();
        h->channel->sent.clear();
    }
    h->view.mm.release();
    // the executor object stays (its manager's staging threads cannot be stopped); the handle with it
}

// What the controller does to an executor (controller.hpp:429-431 -> cuda_server.hpp:282-285):
// returns when the executor's loop has acted on the signal.
void tso_exec_signal(void* hv, int signal, const char* func) {
    string f(func);
    ((ExecHandle*)hv)->ex->sig_exec_from_controller(signal, f);
}

// One serialised QueryList, as the client's sender pushes it (cuda_server.hpp:199-209).  Returns
// when the executor is back at its poll; `out` receives what it sent to its clients meanwhile as
// records of a 4-byte little-endian length followed by the serialised response.  The return value
// is the size the records need.
int tso_exec_queries(void* hv, const void* bytes, int n, void* out, int cap) {
    auto* h = (ExecHandle*)hv;
    std::string msg((const char*)bytes, (size_t)n);
    {   // argument sizes of the launches inside, for the launch recorder
        QueryList ql;
        ql.ParseFromString(msg);
        std::lock_guard<std::mutex> g(g_launch_mu);
        for (auto& q : ql.queries()) {
            if (q.type() != QueryType::cudaLaunchKernel) continue;
            cudaLaunchKernelQuery lq;
            lq.ParseFromString(q.query());
            if (!lookup().count(lq.function())) continue;     // the executor will not launch it
            std::vector<size_t> sizes;
            for (int i = 0; i < lq.args_size(); ++i) sizes.push_back(lq.args(i).length());
            g_expected_arg_sizes.push_back(sizes);
        }
    }
    std::vector<std::string> sent;
    {
        std::unique_lock<std::mutex> lk(h->channel->mu);
        h->channel->inbox.push_back(msg);
        h->channel->cv.notify_all();
        h->channel->cv.wait(lk, [&] { return h->channel->inbox.empty() && !h->channel->busy; });
        sent.swap(h->channel->sent);
    }
    std::string records;
    for (auto& s : sent) {
        uint32_t len = (uint32_t)s.size();
        records.append((const char*)&len, 4);
        records.append(s);
    }
    if (out && (int)records.size() <= cap) memcpy(out, records.data(), records.size());
    return (int)records.size();
}

// Kernel launches the executor made since the last call: one line each, the kernel's name and the
// argument bytes it passed (after its pointer rewrite) in hex.
int tso_exec_launches(char* out, int cap) {
    std::lock_guard<std::mutex> g(g_launch_mu);
    std::string text;
    static const char* hex = "0123456789abcdef";
    for (auto& l : g_launches) {
        text += l.kernel;
        for (auto& a : l.args) {
            text += ' ';
            for (unsigned char c : a) { text += hex[c >> 4]; text += hex[c & 15]; }
            if (a.empty()) text += '-';
        }
        text += '\n';
    }
    const int need = (int)text.size() + 1;
    if (out && need <= cap) {
        memcpy(out, text.c_str(), need);
        g_launches.clear();
    }
    return need;
}

// Executor ids that have reported a finished request to the controller (controller_sync_queue).
int tso_exec_completions(int* out, int cap) {
    int n = 0;
    while (!server::controller_sync_queue->empty()) {
        int id = server::controller_sync_queue->front();
        server::controller_sync_queue->pop();
        if (out && n < cap) out[n] = id;
        ++n;
    }
    return n;
}

void tso_exec_reset(void) {
    std::lock_guard<std::mutex> g(g_launch_mu);
    g_expected_arg_sizes.clear();
    g_launches.clear();
    kernel_model_access_loc().clear();
    while (!server::controller_sync_queue->empty()) server::controller_sync_queue->pop();
}
#endif

}  // extern "C"
