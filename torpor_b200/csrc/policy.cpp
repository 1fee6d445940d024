// Eviction policy of the swap path: which resident models make room for a swap-in.
//
// Same decisions as the reference's LRUEvictor and InterferenceAwareEvictor
// (include/server/evictor.hpp:14-264), kept as recency stamps on flat per-GPU
// tables instead of linked lists: "front of the list" is the largest stamp,
// the eviction scan "from the back" visits entries by increasing stamp.
// Where the reference would spin forever because nothing can be evicted
// (evictor.hpp:84-95,211-224) these return TSW_ERR_STATE and change nothing.

#include "engine.hpp"

#include <algorithm>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

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

}  // namespace

struct tsw_evictor {
    bool lru = true;
    uint64_t budget = 0;
    uint64_t clock = 0;
    std::vector<GpuState> gpu;
    std::unordered_map<std::string, std::set<int>> where;   // IA: model_to_gpus
    std::unordered_map<std::string, int> level;

    // least recently used, unlocked entry of a class (0 = any class)
    const std::string* victim(const GpuState& g, int cls) const {
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
    int choose(const GpuState& g, uint64_t size, const std::vector<int>& class_order, std::vector<std::string>* out) const {
        GpuState probe = g;  // work on a copy: nothing changes unless the request can be satisfied
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

extern "C" {

int tsw_evictor_create(const char* kind, int gpu_count, uint64_t budget, tsw_evictor** out) {
    if (!out || gpu_count <= 0) return tsw::fail(TSW_ERR_INVALID, "bad evictor arguments");
    auto* ev = new tsw_evictor();
    ev->lru = kind && std::string(kind) == "LRU";  // EVICT_POLICY=LRU, else interference-aware (controller.hpp:103-109)
    ev->budget = budget;
    ev->gpu.resize(gpu_count);
    *out = ev;
    return TSW_OK;
}

int tsw_evictor_destroy(tsw_evictor* ev) {
    delete ev;
    return TSW_OK;
}

int tsw_evictor_check_and_add(tsw_evictor* ev, int gpu_idx, const char* func, uint64_t size, int level, char* victims,
                              int cap) {
    if (!ev || !func || gpu_idx < 0 || gpu_idx >= (int)ev->gpu.size()) return tsw::fail(TSW_ERR_INVALID, "bad evictor arguments");
    const std::string f(func);
    ev->level[f] = level;
    GpuState& g = ev->gpu[gpu_idx];
    if (victims && cap > 0) victims[0] = 0;

    // a hit only refreshes recency
    const bool present = ev->lru ? g.items.count(f) > 0 : (ev->where.count(f) && ev->where[f].count(gpu_idx));
    if (present) {
        auto it = g.items.find(f);
        if (it != g.items.end()) it->second.stamp = ++ev->clock;
        return 0;
    }

    std::vector<std::string> out;
    const std::vector<int> order = ev->lru ? std::vector<int>{0} : std::vector<int>{2, 1};
    if (ev->choose(g, size, order, &out) != 0)
        return tsw::fail(TSW_ERR_STATE, "nothing left to evict: every resident model is locked or the model exceeds the budget");
    std::string joined;
    for (size_t i = 0; i < out.size(); ++i) {
        if (i) joined += "\n";
        joined += out[i];
    }
    if (victims && (int)joined.size() + 1 > cap) return tsw::fail(TSW_ERR_BUFFER, "victim buffer too small");

    for (auto& v : out) {
        g.cur -= g.items[v].size;
        g.items.erase(v);
    }
    Entry en;
    en.size = size;
    en.stamp = ++ev->clock;
    if (!ev->lru) {
        auto& homes = ev->where[f];
        if (level >= kLevelMedian && homes.empty()) {
            en.cls = 1;
        } else {
            en.cls = 2;
            if (level >= kLevelMedian) {
                // another replica exists: the former sole replica elsewhere is no longer precious
                for (int other : homes) {
                    auto it = ev->gpu[other].items.find(f);
                    if (it != ev->gpu[other].items.end() && it->second.cls == 1) {
                        it->second.cls = 2;
                        it->second.stamp = ++ev->clock;
                    }
                }
            }
        }
        homes.insert(gpu_idx);
    }
    g.items[f] = en;
    g.cur += size;
    if (!ev->lru) {
        for (auto& v : out) {
            auto& homes = ev->where[v];
            homes.erase(gpu_idx);
            if (ev->level[v] >= kLevelMedian && homes.size() == 1) {
                const int other = *homes.begin();
                auto it = ev->gpu[other].items.find(v);
                if (it != ev->gpu[other].items.end() && it->second.cls == 2) {
                    it->second.cls = 1;
                    it->second.stamp = ++ev->clock;
                }
            }
        }
    }
    if (victims) memcpy(victims, joined.c_str(), joined.size() + 1);
    return (int)out.size();
}

int tsw_evictor_force_evict(tsw_evictor* ev, int gpu_idx, const char* func) {
    if (!ev || !func || gpu_idx < 0 || gpu_idx >= (int)ev->gpu.size()) return tsw::fail(TSW_ERR_INVALID, "bad evictor arguments");
    GpuState& g = ev->gpu[gpu_idx];
    auto it = g.items.find(func);
    if (it != g.items.end()) {
        g.cur -= it->second.size;
        g.items.erase(it);
    }
    if (!ev->lru) {
        auto w = ev->where.find(func);
        if (w != ev->where.end()) w->second.erase(gpu_idx);
    }
    return TSW_OK;
}

int tsw_evictor_lock(tsw_evictor* ev, int gpu_idx, const char* func) {
    if (!ev || !func || gpu_idx < 0 || gpu_idx >= (int)ev->gpu.size()) return tsw::fail(TSW_ERR_INVALID, "bad evictor arguments");
    GpuState& g = ev->gpu[gpu_idx];
    // the LRU policy only locks what it holds (evictor.hpp:246-251); the interference-aware one always locks (:174-176)
    if (!ev->lru || g.items.count(func)) g.locked.insert(func);
    return TSW_OK;
}

int tsw_evictor_unlock(tsw_evictor* ev, int gpu_idx, const char* func) {
    if (!ev || !func || gpu_idx < 0 || gpu_idx >= (int)ev->gpu.size()) return tsw::fail(TSW_ERR_INVALID, "bad evictor arguments");
    ev->gpu[gpu_idx].locked.erase(func);
    return TSW_OK;
}

}  // extern "C"

// =====================================================================================
// Swap scheduler: which GPU runs a request, and where its weights come from.
//
// The decision functions of the reference's controller (include/server/controller.hpp:
// random_schedule :296-318, interference_aware_schedule :321-389, model_level_to_exec_status
// :26-33) for any number of GPUs.  The reference hard-codes a 4-GPU box (pcie_pairs_ and
// nvlink_topology_, :116-118); here both tables are inputs.  With no tables given the
// defaults describe an NVSwitch machine: every peer is a "fast" NVLink neighbour, and GPU i
// shares its PCIe uplink with GPU i^1.
namespace {
constexpr int kAvail = -1, kRunLocal = 0, kRunNvlink = 1, kRunPcieLight = 2, kRunPcieMedian = 3;  // controller.hpp:18-24
}

struct tsw_scheduler {
    int n = 0;
    bool random_policy = false;
    std::vector<int> status;                 // executor_status_[i].status_
    std::vector<int> pcie_pair;
    std::vector<std::vector<int>> nvlink;    // 0 self, 1 slow, 2 fast, -1 PCIe only
    std::unordered_map<std::string, int> level;
};

extern "C" {

int tsw_sched_create(int gpu_count, const char* policy, const int* pcie_pairs, const int* nvlink, tsw_scheduler** out) {
    if (!out || gpu_count <= 0) return tsw::fail(TSW_ERR_INVALID, "bad scheduler arguments");
    auto* s = new tsw_scheduler();
    s->n = gpu_count;
    s->random_policy = policy && std::string(policy) == "RAND";   // SCHEDULE_POLICY=RAND (controller.hpp:95-101)
    s->status.assign(gpu_count, kAvail);
    s->pcie_pair.resize(gpu_count);
    s->nvlink.assign(gpu_count, std::vector<int>(gpu_count, 2));
    for (int i = 0; i < gpu_count; ++i) {
        const int sibling = (i ^ 1) < gpu_count ? (i ^ 1) : i;
        s->pcie_pair[i] = pcie_pairs ? pcie_pairs[i] : sibling;
        if (s->pcie_pair[i] < 0 || s->pcie_pair[i] >= gpu_count) {
            delete s;
            return tsw::fail(TSW_ERR_INVALID, "PCIe sibling out of range");
        }
        for (int j = 0; j < gpu_count; ++j) s->nvlink[i][j] = nvlink ? nvlink[i * gpu_count + j] : (i == j ? 0 : 2);
    }
    *out = s;
    return TSW_OK;
}

int tsw_sched_destroy(tsw_scheduler* s) {
    delete s;
    return TSW_OK;
}

int tsw_sched_set_status(tsw_scheduler* s, int gpu, int status) {
    if (!s || gpu < 0 || gpu >= s->n) return tsw::fail(TSW_ERR_INVALID, "bad scheduler arguments");
    s->status[gpu] = status;
    return TSW_OK;
}

int tsw_sched_set_level(tsw_scheduler* s, const char* func, int level) {
    if (!s || !func) return tsw::fail(TSW_ERR_INVALID, "bad scheduler arguments");
    s->level[func] = level;
    return TSW_OK;
}

int tsw_sched_decide(tsw_scheduler* s, const char* func, int* gpu, int* src_gpu, int* status) {
    if (!s || !func || !gpu || !src_gpu || !status) return tsw::fail(TSW_ERR_INVALID, "bad scheduler arguments");
    *gpu = *src_gpu = *status = -1;
    std::vector<int> avail;
    for (int i = 0; i < s->n; ++i)
        if (s->status[i] == kAvail) avail.push_back(i);
    if (avail.empty()) return TSW_OK;   // caller queues the request (controller.hpp:176-178)

    std::vector<int> homes;             // model_active_device_map_[func], in its iteration order
    {
        int buf[256];
        int n = tsw_repo_active_devices(func, buf, 256);
        for (int i = 0; i < n && i < 256; ++i)
            if (buf[i] >= 0 && buf[i] < s->n) homes.push_back(buf[i]);
    }
    const int lv = s->level.count(func) ? s->level[func] : 0;
    const int pcie_status = (lv >= 0 && lv <= 2) ? lv + kRunPcieLight : kRunPcieMedian;

    for (int g : homes) {
        if (s->status[g] == kAvail) {   // resident and idle: no swap
            *gpu = g;
            *status = kRunLocal;
            return TSW_OK;
        }
    }
    if (s->random_policy) {
        *gpu = avail[rand() % avail.size()];
        *status = pcie_status;
        return TSW_OK;
    }
    if (!homes.empty()) {
        // resident elsewhere: replica swap over NVLink, preferring a fast pair; the scan keeps
        // the LAST idle GPU that has a fast neighbour among the replicas (controller.hpp:346-355)
        int dst = avail[0], src = homes[0];
        for (int gi : avail) {
            for (int gj : homes) {
                if (s->nvlink[gi][gj] == 2) {
                    dst = gi;
                    src = gj;
                    break;
                }
            }
        }
        *gpu = dst;
        *src_gpu = src;
        *status = kRunNvlink;
        return TSW_OK;
    }
    // from the host store: the idle GPU whose PCIe sibling is least busy (:379-385)
    int best = avail[0], best_status = s->status[s->pcie_pair[avail[0]]];
    for (int g : avail) {
        if (s->status[s->pcie_pair[g]] < best_status) {
            best_status = s->status[s->pcie_pair[g]];
            best = g;
        }
    }
    *gpu = best;
    *status = pcie_status;
    return TSW_OK;
}

}  // extern "C"

// Topology tables for the scheduler, read from the machine instead of hard-coded
// (controller.hpp:116-118 has "TODO import function pcie sharing and nvlink topology").
// nvlink[i*n+j]: 0 self, 2 = peer access at the best performance rank (NVLink / NVSwitch),
// 1 = peer access at a lower rank, -1 = no peer access.  pcie_pairs[i]: another GPU below the
// same PCIe root port (they share the uplink to the host), or i itself when it has the port alone.
#include <cuda_runtime.h>
#include <climits>
#include <cstdlib>

extern "C" int tsw_topology_discover(int gpu_count, int* pcie_pairs, int* nvlink) {
    if (gpu_count <= 0 || !pcie_pairs || !nvlink) return tsw::fail(TSW_ERR_INVALID, "bad topology arguments");
    int present = 0;
    cudaError_t err = cudaGetDeviceCount(&present);
    if (err != cudaSuccess || present < gpu_count) {
        cudaGetLastError();
        return tsw::fail(TSW_ERR_NO_DEVICE, "fewer CUDA devices than asked for");
    }
    std::vector<std::string> port(gpu_count);
    for (int i = 0; i < gpu_count; ++i) {
        char bdf[32] = {0};
        if (cudaDeviceGetPCIBusId(bdf, sizeof(bdf), i) != cudaSuccess) continue;
        for (char* c = bdf; *c; ++c) *c = (char)tolower(*c);
        char resolved[PATH_MAX];
        const std::string link = std::string("/sys/bus/pci/devices/") + bdf;
        if (!realpath(link.c_str(), resolved)) continue;
        // /sys/devices/pci0000:15/0000:15:01.0/...: the first two components after /sys/devices name the root port
        std::string p(resolved);
        size_t a = p.find("/pci");
        if (a == std::string::npos) continue;
        size_t b = p.find('/', a + 1);
        size_t c = b == std::string::npos ? b : p.find('/', b + 1);
        port[i] = p.substr(a, (c == std::string::npos ? p.size() : c) - a);
        if (c == std::string::npos) port[i].clear();   // the GPU sits directly on the root bus: nothing to share
    }
    for (int i = 0; i < gpu_count; ++i) {
        pcie_pairs[i] = i;
        for (int j = 0; j < gpu_count; ++j)
            if (j != i && !port[i].empty() && port[i] == port[j]) {
                pcie_pairs[i] = j;
                break;
            }
        for (int j = 0; j < gpu_count; ++j) {
            int v = 0;
            if (i != j) {
                int ok = 0, rank = 0;
                cudaDeviceGetP2PAttribute(&ok, cudaDevP2PAttrAccessSupported, i, j);
                cudaDeviceGetP2PAttribute(&rank, cudaDevP2PAttrPerformanceRank, i, j);
                v = !ok ? -1 : (rank == 0 ? 2 : 1);
            }
            nvlink[i * gpu_count + j] = v;
        }
    }
    return TSW_OK;
}
