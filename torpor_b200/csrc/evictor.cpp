// Eviction policy of the swap path: which resident models make room for a swap-in.
//
// Same decisions as the reference's LRUEvictor and InterferenceAwareEvictor
// (include/server/evictor.hpp:14-264), kept as recency stamps on flat per-GPU
// tables instead of linked lists: "front of the list" is the largest stamp,
// the eviction scan "from the back" visits entries by increasing stamp.
// Where the reference would spin forever because nothing can be evicted
// (evictor.hpp:84-95,211-224) these return TSW_ERR_STATE and change nothing.

#include "policy_internal.hpp"

using namespace tsw_policy;

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
    if (victims && cap > 0) victims[0] = 0;
    std::vector<std::string> out;
    const int rc = evictor_check_and_add(ev, gpu_idx, func, size, level, &out, victims ? cap : -1);
    if (rc < 0) return rc;
    if (victims) {
        size_t at = 0;
        for (size_t i = 0; i < out.size(); ++i) {
            if (i) victims[at++] = '\n';
            memcpy(victims + at, out[i].c_str(), out[i].size());
            at += out[i].size();
        }
        victims[at] = 0;
    }
    return rc;
}

}  // extern "C"

// check_and_add of both policies (evictor.hpp:41-113,196-229).  Returns the number of victims
// (listed in `out`, in eviction order) or a negative status; nothing changes on failure.
// `text_cap` >= 0 refuses, before anything changes, a victim list whose newline-joined text
// would not fit a caller's buffer of that size.  `must_add` is for a model that is on the GPU
// already (a cold start that has just finished): everything unpinned that the scan would take
// is evicted and the model is entered even if the GPU stays over its limit.
int evictor_check_and_add(tsw_evictor* ev, int gpu_idx, const std::string& f, uint64_t size, int level,
                                 std::vector<std::string>* victims, int text_cap, bool must_add) {
    ev->level[f] = level;
    GpuState& g = ev->gpu[gpu_idx];

    // a hit only refreshes recency
    const bool present = ev->lru ? g.items.count(f) > 0 : (ev->where.count(f) && ev->where[f].count(gpu_idx));
    if (present) {
        auto it = g.items.find(f);
        if (it != g.items.end()) it->second.stamp = ++ev->clock;
        return 0;
    }

    std::vector<std::string>& out = *victims;
    const std::vector<int> order = ev->lru ? std::vector<int>{0} : std::vector<int>{2, 1};
    if (ev->choose(g, size, order, &out) != 0 && !must_add) {
        out.clear();
        return tsw::fail(TSW_ERR_STATE, "nothing left to evict: every resident model is locked or the model exceeds the budget");
    }
    if (text_cap >= 0) {
        size_t text = out.empty() ? 0 : out.size() - 1;   // separators
        for (auto& v : out) text += v.size();
        if (text + 1 > (size_t)text_cap) {
            out.clear();
            return tsw::fail(TSW_ERR_BUFFER, "victim buffer too small");
        }
    }

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
    return (int)out.size();
}

extern "C" {

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
