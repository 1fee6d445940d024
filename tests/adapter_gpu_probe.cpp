// The drop-in adapter (torpor_b200/adapter: the reference's MemoryManager class and method names
// over libtorpor_swap.so) on a real GPU, driven as the reference's executor drives the original
// (cuda_server.hpp:73-74,223-253,951-978,1265-1268): cold start, eviction, another function
// taking the freed pool blocks, swap-in by signal, translation of every parameter, and the bytes
// read back from the translated addresses with the plain CUDA runtime.  Compiled where the
// reference's common headers lie (oracle/Makefile, target ref); run by tests/test_gpu_adapter.py.
#include "memory_manager.hpp"
#include "spdlog/sinks/null_sink.h"

#include <cstdio>
#include <cstring>
#include <vector>

namespace {
struct Param { size_t block, offset, size; std::string bytes; void* vptr = nullptr; };

std::string seeded(size_t n, uint64_t seed) {
    std::string s(n, '\0');
    uint64_t x = seed * 0x9E3779B97F4A7C15ull + 1;
    for (size_t i = 0; i < n; ++i) {
        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
        s[i] = (char)(x >> 32);
    }
    return s;
}
}  // namespace

int main() {
    using namespace server;
    using namespace server::manager;
    std::streambuf* console = std::cout.rdbuf(nullptr);       // the adapter's progress lines are not wanted here
    auto log = std::make_shared<spdlog::logger>("probe", std::make_shared<spdlog::sinks::null_sink_mt>());
    MemoryManager mm(0);
    mm.set_logger(log);
    mm.set_server_id(0);
    mm.start_trans_thread(1);
    if (!mm.engine()) { fprintf(stderr, "no engine: %s\n", tsw_last_error()); return 1; }

    const size_t MiB = 1 << 20;
    const std::vector<size_t> block_sizes = {2 * MiB, 20 * MiB, 24 * MiB};
    auto cold_start = [&](string f, uint64_t seed, std::vector<Param>& params) -> int {
        params = {{0, 0, 4096}, {0, 4096, 300000}, {0, 304640, 1000001}, {0, 1305600, 512}, {0, 1306112, 7},
                  {1, 0, 5 * MiB}, {1, 5 * MiB, 9 * MiB + 13}, {2, 0, 24 * MiB}};
        std::vector<void*> blocks;
        mm.set_track_model_memory(f);
        for (size_t b = 0; b < block_sizes.size(); ++b) {
            void* p = mm.cudaMallocBackend(block_sizes[b], true, f);
            if (!p) return 10;
            blocks.push_back(p);
            for (size_t i = 0; i < params.size(); ++i) {
                if (params[i].block != b) continue;
                params[i].bytes = seeded(params[i].size, seed * 100 + i);
                params[i].vptr = (char*)p + params[i].offset;
                mm.cudaMemcpyAsyncBackendHtoD(params[i].vptr, params[i].bytes, nullptr, true, f);
            }
        }
        if (cudaDeviceSynchronize() != cudaSuccess) return 11;
        mm.init_model_readiness(f);
        if (!mm.cudaMallocBackend(2 * MiB, false, f)) return 12;     // a workspace block
        for (auto& p : params)
            if (!mm.try_insert_model_access(p.vptr)) return 13;
        mm.unset_track_model_memory(f);
        return 0;
    };
    auto resident_equal = [&](string f, std::vector<Param>& params, int* moved) -> int {
        std::vector<char> back;
        for (auto& p : params) {
            void* phys = mm.get_cuda_addr(f, p.vptr);
            if (!phys) return 20;
            if (phys != p.vptr && moved) ++*moved;
            back.assign(p.size, 0);
            if (cudaMemcpy(back.data(), phys, p.size, cudaMemcpyDeviceToHost) != cudaSuccess) return 21;
            if (memcmp(back.data(), p.bytes.data(), p.size) != 0) return 22;
        }
        return 0;
    };

    string f = "fn", g = "other";
    std::vector<Param> pf, pg;
    int rc = cold_start(f, 1, pf);
    if (rc) { fprintf(stderr, "cold start of fn: %d (%s)\n", rc, tsw_last_error()); return rc; }
    if ((rc = resident_equal(f, pf, nullptr))) { fprintf(stderr, "fn after its cold start: %d\n", rc); return rc; }
    mm.evict_model(f);
    if (mm.check_model_alloc_status(f)) return 30;
    rc = cold_start(g, 2, pg);                                      // takes the pool blocks fn has just given back
    if (rc) { fprintf(stderr, "cold start of other: %d (%s)\n", rc, tsw_last_error()); return rc; }
    mm.sig_trans_thread(f, -1);                                     // the swap signal: place, rebind, one kernel
    if (!mm.check_model_alloc_status(f)) return 31;
    int moved = 0;
    if ((rc = resident_equal(f, pf, &moved))) { fprintf(stderr, "fn after swap-in: %d (%s)\n", rc, tsw_last_error()); return rc; }
    if (moved == 0) { fprintf(stderr, "fn came back at its old addresses: nothing was rebound\n"); return 32; }
    if ((rc = resident_equal(g, pg, nullptr))) { fprintf(stderr, "other, resident beside fn: %d\n", rc); return rc; }
    // twice more, with the other function leaving and returning in between
    for (int round = 0; round < 2; ++round) {
        mm.evict_model(g);
        mm.evict_model(f);
        mm.sig_trans_thread(g, -1);
        mm.sig_trans_thread(f, -1);
        if ((rc = resident_equal(f, pf, nullptr)) || (rc = resident_equal(g, pg, nullptr))) {
            fprintf(stderr, "round %d: %d (%s)\n", round, rc, tsw_last_error());
            return rc;
        }
    }
    uint64_t launches = 0, bytes = 0, ns = 0;
    tsw_stats(mm.engine(), &launches, &bytes, &ns);
    mm.evict_model(f);
    mm.evict_model(g);
    mm.destroy_trans_thread();
    std::cout.rdbuf(console);
    printf("adapter gpu probe ok: %d parameters rebound, %llu kernel launches, %llu bytes moved\n", moved,
           (unsigned long long)launches, (unsigned long long)bytes);
    return 0;
}
