// Shared between evictor.cpp, scheduler.cpp and controller.cpp: the policy objects behind the opaque
// handles of include/torpor_swap.h.  Not part of the library's interface.
#ifndef TSW_POLICY_INTERNAL_HPP_
#define TSW_POLICY_INTERNAL_HPP_

#include "engine.hpp"

#include <algorithm>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace tsw_policy {

constexpr int kLevelMedian = 1;  // ModelLevel_Median (evictor.hpp:10-12)

struct Entry {
    uint64_t size = 0;
    uint64_t stamp = 0;
    int cls = 2;  // IA: 1 = first class (sole replica of a non-light model), 2 = second class
};

struct GpuState {
    std::unordered_map<std::string, Entry> items;
    std::unordered_set<std::string> locked;
    uint64_t cur = 0;
};


constexpr int kAvail = -1, kRunLocal = 0, kRunNvlink = 1, kRunPcieLight = 2, kRunPcieMedian = 3;  // controller.hpp:18-24

}  // namespace tsw_policy

struct tsw_evictor {
    bool lru = true;
    uint64_t budget = 0;
    uint64_t clock = 0;
    std::vector<tsw_policy::GpuState> gpu;
    std::unordered_map<std::string, std::set<int>> where;   // IA: model_to_gpus
    std::unordered_map<std::string, int> level;

    // least recently used, unlocked entry of a class (0 = any class)
    const std::string* victim(const tsw_policy::GpuState& g, int cls) const {
        const std::string* best = nullptr;
        uint64_t best_stamp = ~0ull;
        for (auto& kv : g.items) {
            if (cls && kv.second.cls != cls) continue;
            if (g.locked.count(kv.first)) continue;
            if (kv.second.stamp < best_stamp) {
                best_stamp = kv.second.stamp;
                best = &kv.first;
            }
        }
        return best;
    }

    // Pick victims until `size` fits, first from `order[0]`, then `order[1]`...; -1 if it cannot fit.
    int choose(const tsw_policy::GpuState& g, uint64_t size, const std::vector<int>& class_order, std::vector<std::string>* out) const {
        tsw_policy::GpuState probe = g;  // work on a copy: nothing changes unless the request can be satisfied
        for (int cls : class_order) {
            while (probe.cur + size >= budget) {  // `>=` as in evictor.hpp:65,85,211
                const std::string* v = victim(probe, cls);
                if (!v) break;
                out->push_back(*v);
                probe.cur -= probe.items[*v].size;
                probe.items.erase(*v);
            }
        }
        return probe.cur + size >= budget ? -1 : 0;
    }
};

struct tsw_scheduler {
    int n = 0;
    bool random_policy = false;
    std::vector<int> status;                 // executor_status_[i].status_
    std::vector<int> pcie_pair;
    std::vector<std::vector<int>> nvlink;    // 0 self, 1 slow, 2 fast, -1 PCIe only
    std::unordered_map<std::string, int> level;
};

// check_and_add of both policies with the victims as a list (evictor.cpp); the controller calls it directly.
int evictor_check_and_add(tsw_evictor* ev, int gpu_idx, const std::string& f, uint64_t size, int level,
                          std::vector<std::string>* victims, int text_cap, bool must_add = false);

#endif  // TSW_POLICY_INTERNAL_HPP_
