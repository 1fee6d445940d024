// Host model store and address-translation tables of the swap engine.
//
// Holds what the reference keeps in ModelRepo (include/server/model_repo.hpp:12-186)
// -- per function: the client's device blocks, the parameters uploaded into them,
// the authoritative host copy and the first-run access order; per (GPU, function):
// where every block and parameter currently lives -- as flat, index-linked arrays.
// The host copy is page-locked, device-mapped memory so that the placement kernel
// can read it in place; the reference keeps it pageable and stages it through a
// pinned mirror on every swap (model_repo.hpp:173-177, memory_manager.hpp:311-329).
#ifndef TORPOR_SWAP_REPO_HPP_
#define TORPOR_SWAP_REPO_HPP_

#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

struct tsw_engine;

namespace tsw {

struct VBlock {                 // GeneralBlockInfo + ModelBlockInfo (model_repo.hpp:12-23)
    uint64_t vaddr = 0;         // client-visible device pointer (= first placement)
    uint64_t canon = 0;         // the same in the canonical address space (table key)
    uint64_t size = 0;
    bool is_model = false;
    bool alive = true;
    uint8_t* mirror = nullptr;  // host copy of a model block
    bool mirror_heap = false;   // mirror came from malloc (plan-only engines)
    std::vector<int> params;    // parameters uploaded into this block
    std::vector<uint64_t> ephe; // interior pointers cached for this block
};

struct VParam {                 // ModelParamInfo (model_repo.hpp:25-30)
    uint64_t vaddr = 0;
    uint64_t size = 0;
    int block = -1;
    uint64_t canon = 0;         // vaddr in the canonical address space
    uint8_t* host = nullptr;    // inside the block's mirror
    bool accessed = false;
};

// Per (engine, function) placement: DeviceModelInfo (model_repo.hpp:48-65) plus the
// readiness map the reference keeps in the manager (memory_manager.hpp:33,590).
struct Placement {
    int status = 1;  // TSW_MODEL_INCOMPLETE until the controller marks it (model_repo.hpp:64)
    struct B { bool known = false, in_cuda = false; uint64_t cuda = 0, canon = 0; };
    struct P { bool known = false; uint64_t cuda = 0, canon = 0; };
    std::vector<B> blocks;
    std::vector<P> params;
    bool readiness_init = false;
    // Pointer-table columns, one row per parameter.  On a CUDA engine they are
    // host-mapped page-locked arrays written by the placement kernel; on a plan-only
    // engine plain memory written by the planner.
    uint32_t capacity = 0;
    bool counters_dirty = false;         // a swap ended with rows incomplete: their tile counters hold partial counts
    std::vector<void*> retired_rows;     // plan-only: smaller tables replaced by growth; a waiter may still read them
    volatile uint32_t* flag = nullptr;   // TSW_READY_*
    volatile uint64_t* phys = nullptr;   // readiness address (0 = none)
    // Generation word per row, host-mapped like the two columns above: the swap generation that last
    // completed the row.  Stream-ordered waits (tsw_translate_async) wait on THIS word, because it is
    // the one the host can write with a plain store when a wait has to be let go: a release that went
    // through a CUDA stream could be queued by the driver behind the very wait it is meant to end.
    volatile uint32_t* gen = nullptr;
    std::vector<bool> has_row;           // row exists in the readiness map
    // device-side twins and launch scratch (CUDA engines only)
    uint64_t* d_table_phys = nullptr;
    uint32_t* d_table_flag = nullptr;
    uint32_t* d_done = nullptr;
    uint32_t* d_ticket = nullptr;   // tile dispenser of sharded swaps
    void* d_descs = nullptr;
    uint32_t* d_first = nullptr;
    void* h_descs = nullptr;
    uint32_t* h_first = nullptr;
    bool in_flight = false;
    // Swap generation.  The device flag column holds the generation that last completed a row
    // (never a plain "ready"), so that a stream-ordered wait enqueued for generation g cannot be
    // satisfied by what an earlier swap left behind.  Starts at 2 and only grows.
    uint32_t epoch = 1;
    std::vector<tsw_engine*> helpers;   // engines whose kernels still write into these blocks
    std::vector<int> remote_rows;       // rows handed out by a plan and not yet committed
    // Stream-ordered waits (tsw_translate_async) enqueued for rows of the current generation, and
    // rows whose waiters were let go without their bytes: translation and polling report those as
    // failed until the model is swapped in again or evicted.
    std::vector<int> waited_rows;
    std::vector<bool> failed;
};

struct Model {                  // HostModelInfo (model_repo.hpp:37-46)
    std::string name;
    int status = 1;             // TSW_MODEL_INCOMPLETE
    uint64_t total_size = 0;
    std::vector<VBlock> blocks;
    std::vector<VParam> params;
    // Iteration order of the reference's pointer-keyed block map; swap-in requests
    // pool blocks, and evict releases them, in this order (memory_manager.hpp:461,247).
    std::unordered_map<void*, int> block_order;
    std::unordered_map<uint64_t, int> block_by_vaddr;
    std::unordered_map<uint64_t, int> param_by_vaddr;
    std::unordered_map<uint64_t, int> data_block;   // virtual_data_block_mapping_: pointer -> block
    std::vector<int> access_order;                   // model_access_order_map_
    bool has_access_order = false;
    std::map<int, Placement> place;                  // by server id
};

struct Repo {
    std::recursive_mutex mu;
    std::unordered_map<std::string, std::unique_ptr<Model>> models;
    // model_active_device_map_: hashed like the reference's, whose scheduler walks it in hash order
    std::unordered_map<std::string, std::unordered_set<int>> active_devices;

    Model* find(const std::string& f) {
        auto it = models.find(f);
        return it == models.end() ? nullptr : it->second.get();
    }
    Model* get_or_create(const std::string& f) {
        auto& m = models[f];
        if (!m) { m.reset(new Model()); m->name = f; }
        return m.get();
    }
};

Repo& repo();

}  // namespace tsw
#endif
