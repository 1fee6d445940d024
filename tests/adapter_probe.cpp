// Compile-and-run probe for torpor_b200/adapter: uses the drop-in headers exactly as the
// reference's executor and controller use the originals (cuda_server.hpp:50,73-74,106,223-253,
// 951-978; controller.hpp:103-109,392-400), on a plan-only engine so that no GPU is needed.
#include "memory_manager.hpp"
#include "evictor.hpp"
#include "spdlog/sinks/null_sink.h"
#include "spdlog/sinks/ostream_sink.h"

#include <sstream>

#include <cstdio>
#include <cstring>

int main() {
    using namespace server;
    using namespace server::manager;
    setenv("TORPOR_SWAP_ADAPTER_PROBE", "1", 1);
    setenv("TORPOR_SWAP_WAIT_PERIODS", "2", 1);   // bound the repeated wait (unbounded by default, as the reference)
    setenv("TORPOR_SWAP_WAIT_MS", "20", 1);
    auto log = std::make_shared<spdlog::logger>("probe", std::make_shared<spdlog::sinks::null_sink_mt>());
    // the probe drives a plan-only engine directly; start_trans_thread would need a GPU
    tsw_config cfg;
    tsw_config_default(&cfg);
    cfg.device = -1;
    cfg.budget_bytes = 0;
    tsw_engine* e = nullptr;
    if (tsw_engine_create(&cfg, &e) != TSW_OK) return 1;

    string f = "fn";
    uint64_t blk = 0;
    tsw_track_begin(e, f.c_str());
    tsw_malloc(e, f.c_str(), 2 << 20, 1, &blk);
    std::string payload(4096, 'x');
    if (tsw_memcpy_h2d_model(e, f.c_str(), blk + 512, payload.data(), payload.size(), nullptr) != TSW_OK) return 2;
    tsw_sync_done(e, f.c_str());
    tsw_mark_access(e, blk + 512);
    tsw_track_end(e, f.c_str());
    tsw_evict(e, f.c_str(), 0);
    if (tsw_swap_in(e, f.c_str(), -1) != TSW_OK) return 3;
    uint64_t out = 0;
    if (tsw_translate(e, f.c_str(), blk + 512, 1, 1000000, &out) != TSW_OK || out == 0) return 4;

    ModelRepo& repo = ModelRepo::getInstance();
    repo.add_model_info(f, 0);
    if (repo.model_active_device_map_[f].count(0) != 1 || tsw_repo_model_status(f.c_str(), 0) != TSW_MODEL_FULL) return 5;
    repo.remove_model_info(f, 0);
    if (repo.device_model_info_map_[0][f].status_ != ModelStatus_NoData) return 6;

    // the class itself must at least construct and type-check against the executor's calls
    MemoryManager mm(0);
    mm.set_logger(log);
    mm.set_server_id(0);
    void* (MemoryManager::*malloc_fn)(size_t, bool, string&) = &MemoryManager::cudaMallocBackend;
    void (MemoryManager::*sig_fn)(string&, int) = &MemoryManager::sig_trans_thread;
    void* (MemoryManager::*addr_fn)(string&, void*, bool) = &MemoryManager::get_cuda_addr;
    void (MemoryManager::*h2d_fn)(void*, const string&, cudaStream_t, bool, string&) = &MemoryManager::cudaMemcpyAsyncBackendHtoD;
    (void)malloc_fn; (void)sig_fn; (void)addr_fn; (void)h2d_fn;

    // ... and run as the executor runs it (cuda_server.hpp:73-74,223-253,951-978), on a plan-only engine, with
    // a logger that keeps the text: the reference's three timing lines must come out under their own names
    tsw_engine_destroy(e);
    e = nullptr;
    tsw_repo_reset();
    {
        std::ostringstream text;
        auto keep = std::make_shared<spdlog::logger>("probe2", std::make_shared<spdlog::sinks::ostream_sink_mt>(text));
        setenv("TORPOR_SWAP_DEVICE", "-1", 1);
        MemoryManager m2(0);
        m2.set_logger(keep);
        m2.set_server_id(0);
        m2.start_trans_thread(1);
        if (!m2.engine()) return 10;
        string g = "fn2";
        m2.set_track_model_memory(g);
        void* block = m2.cudaMallocBackend(2 << 20, true, g);
        if (!block) return 11;
        m2.cudaMemcpyAsyncBackendHtoD((char*)block + 1024, payload, nullptr, true, g);
        m2.init_model_readiness(g);
        if (!m2.try_insert_model_access((char*)block + 1024)) return 12;
        m2.unset_track_model_memory(g);
        m2.evict_model(g);
        if (m2.check_model_alloc_status(g)) return 13;
        m2.sig_trans_thread(g, -1);
        if (!m2.check_model_alloc_status(g)) return 14;
        if (m2.get_cuda_addr(g, (char*)block + 1024) == nullptr) return 15;
        keep->flush();
        const std::string logged = text.str();
        for (const char* want : {"Evict model fn2 elasped ", "CheckMalloc model fn2 elasped ", "Start transfering model fn2 from GPU -1",
                                 "Transfer model fn2 from -1 wait count 0 pinned elasped 0 overall elasped "})
            if (logged.find(want) == std::string::npos) {
                printf("missing log line: %s\n--- log ---\n%s\n", want, logged.c_str());
                return 16;
            }
        // The wait that runs out: a planned swap whose moves nobody carries out leaves the rows
        // unready.  The reference would block; the adapter repeats the wait a bounded number of
        // periods here and must then answer null -- never the client's own pointer, which names
        // pool memory that may belong to another function by now.
        m2.evict_model(g);
        tsw_segment segs[4];
        tsw_publish pub;
        uint32_t tile = 0;
        if (tsw_swap_plan(m2.engine(), g.c_str(), segs, 4, &tile, &pub) != 1) return 17;
        void* got = m2.get_cuda_addr(g, (char*)block + 1024);
        if (got != nullptr) {
            printf("timed-out translation returned %p (client pointer %p)\n", got, (char*)block + 1024);
            return 18;
        }
        if (tsw_swap_commit(m2.engine(), g.c_str()) != TSW_OK) return 19;
        if (m2.get_cuda_addr(g, (char*)block + 1024) == nullptr) return 20;
        m2.destroy_trans_thread();
    }

    std::shared_ptr<Evictor> ev = std::make_shared<LRUEvictor>(2, 1000);
    map<string, int> levels;
    string a = "a", b = "b", c = "c";
    ev->check_and_add(0, a, 400, levels);
    ev->check_and_add(0, b, 400, levels);
    auto victims = ev->check_and_add(0, c, 400, levels);
    if (victims.size() != 1 || victims[0] != "a") return 7;

    printf("adapter probe ok\n");
    return 0;
}
