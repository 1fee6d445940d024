// Shared between the translation units of the swap engine (engine.cpp, engine_swap.cpp,
// engine_share.cpp): process-wide state and the helpers that more than one of them uses.
// Not part of the library's interface.
#ifndef TSW_ENGINE_INTERNAL_HPP_
#define TSW_ENGINE_INTERNAL_HPP_

#include "engine.hpp"
#include "kernels.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>

#include <cuda_runtime.h>

#define TSW_CUDA(call)                                                                             \
    do {                                                                                           \
        cudaError_t _e = (call);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return fail(TSW_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(_e));         \
    } while (0)

namespace tsw {

extern std::mutex g_engines_mu;
extern std::map<int, tsw_engine*> g_engines;  // server id -> engine of this process

using Lock = std::lock_guard<std::recursive_mutex>;

int64_t now_ns();
Placement& placement(Model* m, int server_id);
void size_placement(Model* m, Placement& pl);
int ensure_rows(tsw_engine* e, Model* m, Placement& pl);             // room for one pointer-table row per parameter
void set_row(Placement& pl, int idx, uint32_t flag, uint64_t phys);
inline uint32_t row_flag(const Placement& pl, int idx) {
    return __atomic_load_n(const_cast<const uint32_t*>(&pl.flag[idx]), __ATOMIC_ACQUIRE);
}
int init_readiness(tsw_engine* e, Model* m, Placement& pl, uint32_t flag);
uint8_t* alloc_mirror(tsw_engine* e, uint64_t size);
uint64_t host_dev_addr(tsw_engine* owner, const uint8_t* p);         // device-visible address of a byte of the host store
bool cache_interior_pointer(Model* m, uint64_t addr);
uint64_t phy_address(tsw_engine* e, Model* m, uint64_t ptr, bool search_amid);

struct WaitResult { int rc; uint64_t phys; };
WaitResult wait_row(tsw_engine* e, Placement& pl, int idx, int64_t timeout_ns);

void* map_shared_far(int fd, uint64_t size, int slot);
int make_arena(tsw_engine* e);
tsw_engine* engine_of_block_mirror(const uint8_t* p);
int place_blocks(tsw_engine* e, Model* m, Placement& pl);
int ensure_peer(tsw_engine* e, int to_device);
int ensure_ce_stream(tsw_engine* e);
uint32_t pick_tile(tsw_engine* e, bool host_side);
int pick_mover(const tsw_engine* e, const std::vector<PlaceDesc>& descs);

struct Plan {
    std::vector<PlaceDesc> descs;
    std::vector<uint32_t> first;  // n + 1
    uint64_t bytes = 0;
};

void finish_plan(Plan& p, uint32_t tile);
int upload_plan(tsw_engine* e, Placement& pl, const Plan& p);

}  // namespace tsw

#endif  // TSW_ENGINE_INTERNAL_HPP_
