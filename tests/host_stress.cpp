// Host-side stress of the swap library under sanitizers (no GPU): several executor threads,
// each with its own plan-only engine, hammer the shared repository concurrently -- cold
// starts, evictions, swap-ins from the host store and from another engine's replica,
// pointer translation with bounded waits, frees and re-mallocs, the eviction policy, the
// scheduler and the controller's request handling.  Built by tests/test_sanitizers.py from the library's host sources with
// -fsanitize=address,undefined or -fsanitize=thread; the kernels' launchers are stubbed.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../include/torpor_swap.h"
#include "../torpor_b200/csrc/kernels.hpp"

namespace tsw {
cudaError_t launch_place(const PlaceArgs&, int, cudaStream_t, int) { return cudaErrorNotSupported; }
cudaError_t launch_publish_rows(const PlaceArgs&, uint32_t, uint32_t, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_checksum(const SumDesc*, uint32_t, uint32_t, uint32_t, unsigned long long*, int, cudaStream_t) { return cudaErrorNotSupported; }
int default_grid_ctas(int) { return 1; }
int default_grid_ctas_host(int) { return 1; }
}  // namespace tsw
extern "C" int tsw_place_segments_static(int, const tsw_segment*, int, uint32_t, uint32_t, uint32_t, const tsw_publish*, void*) { return TSW_ERR_NO_DEVICE; }

static std::atomic<int> g_fail{0};
#define CHECK(x) do { if (!(x)) { fprintf(stderr, "CHECK failed: %s (%s:%d): %s\n", #x, __FILE__, __LINE__, tsw_last_error()); g_fail++; } } while (0)

static void executor(int id, int n_threads, int rounds) {
    tsw_config cfg;
    tsw_config_default(&cfg);
    cfg.device = -1;
    cfg.server_id = id;
    cfg.gpu_count = n_threads;
    cfg.budget_bytes = 0;
    tsw_engine* e = nullptr;
    CHECK(tsw_engine_create(&cfg, &e) == TSW_OK);
    std::vector<std::string> mine;
    std::vector<std::vector<uint64_t>> params;
    const uint64_t sizes[] = {2ull << 20, 20ull << 20, 2ull << 20, 48ull << 20, 130ull << 20};
    for (int k = 0; k < 4; ++k) {
        std::string f = "t" + std::to_string(id) + "_m" + std::to_string(k);
        CHECK(tsw_track_begin(e, f.c_str()) == TSW_OK);
        std::vector<uint64_t> ps;
        for (int b = 0; b < 3 + k; ++b) {
            uint64_t blk = 0;
            CHECK(tsw_malloc(e, f.c_str(), sizes[(b + k) % 5], 1, &blk) == TSW_OK);
            std::string payload(1000 + 37 * b, (char)('a' + b));
            for (int p = 0; p < 3; ++p) {
                uint64_t dst = blk + 4096 * p;
                CHECK(tsw_memcpy_h2d_model(e, f.c_str(), dst, payload.data(), payload.size(), nullptr) == TSW_OK);
                ps.push_back(dst);
            }
        }
        CHECK(tsw_sync_done(e, f.c_str()) == TSW_OK);
        uint64_t ws = 0;
        CHECK(tsw_malloc(e, f.c_str(), 2ull << 20, 0, &ws) == TSW_OK);
        for (size_t i = 0; i < ps.size(); i += 2) CHECK(tsw_mark_access(e, ps[i]) == 1);
        CHECK(tsw_track_end(e, f.c_str()) == TSW_OK);
        tsw_repo_add_model_info(f.c_str(), id);
        mine.push_back(f);
        params.push_back(ps);
        if (k == 1) CHECK(tsw_free(e, f.c_str(), ws) == TSW_OK);
    }
    for (int r = 0; r < rounds; ++r) {
        const int k = (r * 7 + id) % 4;
        const std::string& f = mine[k];
        CHECK(tsw_evict(e, f.c_str(), 0) == TSW_OK);
        tsw_repo_remove_model_info(f.c_str(), id);
        // another thread's model: replica swap if it is marked healthy there, else host store
        const int other = (id + 1 + r) % n_threads;
        std::string of = "t" + std::to_string(other) + "_m" + std::to_string(r % 4);
        // only once its owner has finished loading it (the controller never swaps a model that is
        // still being cold-started): the owner marks it on the repository after track_end
        const bool loaded = tsw_repo_model_status(of.c_str(), other) >= 0 && tsw_repo_total_size(of.c_str()) > 0 &&
                            tsw_repo_model_status(of.c_str(), other) != TSW_MODEL_INCOMPLETE;
        int rc = loaded ? tsw_swap_in(e, of.c_str(), other) : TSW_ERR_UNKNOWN_MODEL;
        if (rc == TSW_OK) {
            CHECK(tsw_wait_ready(e, of.c_str(), 2000000000ll) == TSW_OK);
            CHECK(tsw_check_alloc(e, of.c_str()) == 1);
            CHECK(tsw_evict(e, of.c_str(), 0) == TSW_OK);
        } else {
            CHECK(rc == TSW_ERR_UNKNOWN_MODEL);   // the other thread has not created it yet
        }
        CHECK(tsw_swap_in(e, f.c_str(), -1) == TSW_OK);
        for (uint64_t p : params[k]) {
            uint64_t out = 0;
            CHECK(tsw_translate(e, f.c_str(), p, 1, 1000000000ll, &out) == TSW_OK);
            CHECK(out != 0);
        }
        uint64_t rows[4096];
        CHECK(tsw_dump_params(e, f.c_str(), 1, rows, 4096 / 7) > 0);
        tsw_repo_add_model_info(f.c_str(), id);
        int gpus[16];
        tsw_repo_active_devices(f.c_str(), gpus, 16);
    }
    CHECK(tsw_engine_destroy(e) == TSW_OK);
}

static void policy(int rounds) {
    tsw_evictor* ev = nullptr;
    CHECK(tsw_evictor_create("IA", 4, 1000, &ev) == TSW_OK);
    tsw_scheduler* s = nullptr;
    CHECK(tsw_sched_create(4, "IA", nullptr, nullptr, &s) == TSW_OK);
    char buf[4096];
    for (int r = 0; r < rounds * 20; ++r) {
        std::string f = "p" + std::to_string(r % 11);
        int n = tsw_evictor_check_and_add(ev, r % 4, f.c_str(), 100 + 13 * (r % 7), r % 3, buf, sizeof(buf));
        CHECK(n >= 0);
        if (r % 5 == 0) tsw_evictor_lock(ev, r % 4, f.c_str());
        if (r % 5 == 3) tsw_evictor_unlock(ev, (r - 3) % 4, ("p" + std::to_string((r - 3) % 11)).c_str());
        if (r % 9 == 0) tsw_evictor_force_evict(ev, r % 4, f.c_str());
        int g, src, st;
        tsw_sched_set_level(s, f.c_str(), r % 3);
        CHECK(tsw_sched_decide(s, f.c_str(), &g, &src, &st) == TSW_OK);
        if (g >= 0) tsw_sched_set_status(s, g, r % 2 ? st : -1);
    }
    tsw_evictor_destroy(ev);
    tsw_sched_destroy(s);
}

// The controller's request handling, closed-loop, on its own thread (a controller is driven from one
// thread; what it shares with the executors is the repository, which has its lock).
struct CtrlSink {
    std::vector<int> busy = std::vector<int>(4, 0);
    long signals = 0, acks = 0;
};
static void on_signal(void* user, int gpu, int signal, const char* func) {
    CtrlSink* k = (CtrlSink*)user;
    k->signals++;
    if (gpu < 0 || gpu >= 4 || !func) g_fail++;
    if (signal == TSW_SIGNAL_STARTUP || signal == TSW_SIGNAL_EXECUTE) k->busy[gpu] = 1;
}
static void on_ack(void* user, int, int) { ((CtrlSink*)user)->acks++; }

static void controller(int rounds) {
    tsw_config cfg;
    tsw_config_default(&cfg);
    cfg.device = -1;
    cfg.server_id = 8;
    cfg.gpu_count = 4;
    cfg.budget_bytes = 0;
    tsw_engine* e = nullptr;
    CHECK(tsw_engine_create(&cfg, &e) == TSW_OK);
    for (int i = 0; i < 9; ++i) {            // sizes for the eviction policy: 16..144 MiB of blocks per model
        std::string f = "c" + std::to_string(i);
        uint64_t p;
        tsw_track_begin(e, f.c_str());
        for (int b = 0; b <= i; ++b) CHECK(tsw_malloc(e, f.c_str(), 16ull << 20, 1, &p) == TSW_OK);
        tsw_track_end(e, f.c_str());
    }
    CtrlSink sink;
    tsw_controller* c = nullptr;
    CHECK(tsw_ctrl_create(4, 400ull << 20, "IA", "IA", nullptr, nullptr, on_signal, on_ack, &sink, &c) == TSW_OK);
    unsigned x = 12345;
    auto rnd = [&x]() { x = x * 1664525u + 1013904223u; return x >> 8; };
    for (int r = 0; r < rounds * 40; ++r) {
        std::string f = "c" + std::to_string(rnd() % 9);
        const unsigned pick = rnd() % 100;
        int rc = TSW_OK;
        if (r < 9) rc = tsw_ctrl_request(c, TSW_REQ_EXECUTE_AFTER_LOAD, ("c" + std::to_string(r)).c_str(), std::to_string(r % 4).c_str());
        else if (pick < 50) rc = tsw_ctrl_request(c, TSW_REQ_EXECUTE, f.c_str(), "");
        else if (pick < 88) {
            const int g = (int)(rnd() % 4);
            if (sink.busy[g]) { sink.busy[g] = 0; rc = tsw_ctrl_complete(c, g); }
        } else if (pick < 94) rc = tsw_ctrl_request(c, TSW_REQ_UNLOAD, f.c_str(), pick % 2 ? "" : std::to_string(rnd() % 4).c_str());
        else if (pick < 97) rc = tsw_ctrl_request(c, TSW_REQ_EXECUTE, f.c_str(), std::to_string(rnd() % 4).c_str());
        else rc = tsw_ctrl_request(c, 11 /* Replay: not the controller's */, f.c_str(), "x");
        CHECK(rc == TSW_OK || rc == TSW_ERR_STATE);
        int st;
        char name[64];
        CHECK(tsw_ctrl_executor_status(c, (int)(rnd() % 4), &st, name, sizeof(name)) == TSW_OK);
        int helpers[8];
        CHECK(tsw_ctrl_helpers(c, (int)(rnd() % 4), r % 2, helpers, 8) >= 0);
    }
    for (int g = 0; g < 4; ++g)
        while (sink.busy[g]) { sink.busy[g] = 0; tsw_ctrl_complete(c, g); }
    CHECK(sink.signals > 0 && sink.acks > 0);
    CHECK(tsw_ctrl_queue_depth(c) >= 0);
    tsw_ctrl_destroy(c);
    CHECK(tsw_engine_destroy(e) == TSW_OK);
}

int main(int argc, char** argv) {
    const int n_threads = 4, rounds = argc > 1 ? atoi(argv[1]) : 40;
    std::vector<std::thread> th;
    for (int i = 0; i < n_threads; ++i) th.emplace_back(executor, i, n_threads, rounds);
    th.emplace_back(policy, rounds);
    th.emplace_back(controller, rounds);
    for (auto& t : th) t.join();
    tsw_repo_reset();
    if (g_fail.load()) {
        fprintf(stderr, "host stress: %d checks failed\n", g_fail.load());
        return 1;
    }
    printf("host stress ok\n");
    return 0;
}
