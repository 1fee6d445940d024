// The swap engine: one per GPU, the counterpart of the reference's
// server::manager::MemoryManager (include/server/memory_manager.hpp:36-598).
#ifndef TORPOR_SWAP_ENGINE_HPP_
#define TORPOR_SWAP_ENGINE_HPP_

#include <atomic>
#include <map>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../include/torpor_swap.h"
#include "pool.hpp"
#include "repo.hpp"

namespace tsw {

int fail(int code, const std::string& msg);
const std::string& last_error();

// Bump allocator over one allocation; rows of the pointer table and launch
// descriptors are carved from two of these (device, host-mapped) so that a swap
// never calls the CUDA allocator.
struct Slab {
    uint8_t* base = nullptr;
    uint64_t size = 0, used = 0;
    void* take(uint64_t n, uint64_t align = 256) {
        uint64_t off = (used + align - 1) / align * align;
        if (off + n > size) return nullptr;
        used = off + n;
        return base + off;
    }
};

struct HostArena {
    uint8_t* base = nullptr;      // host address
    int64_t dev_delta = 0;        // device-visible address = host address + dev_delta
    uint64_t size = 0, used = 0;
    std::string shm_name;
    int shm_fd = -1;
    bool owner = false;
    bool anon = false;            // anonymous mapping registered with the driver (huge-page mode)
    bool huge = false;            // the kernel accepted the transparent-huge-page advice
};

}  // namespace tsw

struct tsw_engine {
    tsw_config cfg;
    bool plan = false;
    int server_id = 0;
    std::unique_ptr<tsw::DeviceMemory> mem;
    std::unique_ptr<tsw::Pool> pool;
    std::recursive_mutex mu;

    // set_track_model_memory state (memory_manager.hpp:576)
    bool tracking = false;
    std::string track_func;
    // active_model_params_ (:591): parameters of the model swapped in last
    std::unordered_set<uint64_t> active_params;

    void* stream = nullptr;       // transfer stream (cudaStream_t), high priority
    void* stream_ce = nullptr;    // second transfer stream, made on first use: copy-engine moves of mover 2
    void* ev_ce = nullptr;        // joins stream_ce back into the transfer stream
    void* stage_buf = nullptr;    // tsw_place_segments_pipelined: this GPU's share of a swap while it is on its way
    uint64_t stage_cap = 0;
    void* ev_start = nullptr;     // cudaEvent_t pair around the last swap
    void* ev_stop = nullptr;
    bool ev_valid = false;
    tsw::Slab dev_slab, host_slab;
    uint64_t dev_slab_floor = 0, host_slab_floor = 0;   // what the engine itself took at creation
    tsw::HostArena arena;
    uint32_t* d_status = nullptr;
    volatile uint32_t* h_status = nullptr;

    int grid_ctas = 0;
    int grid_host = 0;   // CTAs of single-GPU launches with one end in the host store (PCIe-bound)
    int grid_bulk = 0;   // CTAs of the bulk-copy mover
    int mover = 0;       // 0 = load/store kernel, 1 = bulk-copy kernel where alignment allows,
                         // 2 = load/store kernel + the copy engine for large parameters read from the host store
    uint64_t ce_min_bytes = 4ull << 20;   // mover 2: parameters of at least this size go to the copy engine
    bool guard_names = false;   // TORPOR_SWAP_GUARD_NAMES=1: never grant an address that names another live block of the model
    uint32_t tile_host = 0, tile_dev = 0;
    int host_store_mode = 0;     // TSW_STORE_*
    uint32_t ticket_chunk = 1;   // tiles per draw from the shared counter of a sharded swap
    std::unordered_set<int> peers;   // devices this engine's device has been given peer access to
    uint32_t last_kernel_status = 0; // last non-zero status word a kernel of this engine reported

    std::atomic<uint64_t> kernel_launches{0};
    std::atomic<uint64_t> bytes_moved{0};
    std::vector<void*> loose_host;   // page-locked mirrors outside the arena

    std::map<std::string, uint64_t> ipc_open;            // IPC handle bytes -> address mapped here
    struct Attached { void* host; uint64_t size; uint64_t dev; };
    std::vector<Attached> attached;                      // shared host arenas registered here

    // launch scratch of tsw_place_segments
    void* raw_d_descs = nullptr;
    void* raw_d_first = nullptr;
    void* raw_h = nullptr;
    uint64_t raw_cap = 0;
};

#endif
