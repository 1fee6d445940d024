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
#include <memory>
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

static int evictor_check_and_add(tsw_evictor* ev, int gpu_idx, const std::string& f, uint64_t size, int level,
                                 std::vector<std::string>* victims, int text_cap, bool must_add = false);

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
static int evictor_check_and_add(tsw_evictor* ev, int gpu_idx, const std::string& f, uint64_t size, int level,
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

// GPUs whose PCIe link carries no swap right now and could lend it to a swap-in of `dst` from
// the host store (tsw_swap_in_sharded).  The signal is the one interference_aware_schedule reads
// (:379-385): an executor status of RunPcie* or RunColdStart means "link busy".  A GPU is left
// out when the GPU it shares an uplink with (pcie_pairs) is `dst`, is loading over PCIe itself,
// or has already been picked -- two GPUs behind one uplink move no more than one.
int tsw_sched_helpers(tsw_scheduler* s, int dst, int include_running, int* helpers, int cap) {
    if (!s || dst < 0 || dst >= s->n || (cap > 0 && !helpers)) return tsw::fail(TSW_ERR_INVALID, "bad scheduler arguments");
    auto link_busy = [&](int g) { return s->status[g] >= kRunPcieLight; };
    std::vector<char> taken(s->n, 0);
    taken[dst] = 1;
    int n = 0;
    for (int g = 0; g < s->n; ++g) {
        if (g == dst) continue;
        const bool idle = s->status[g] == kAvail || (include_running && !link_busy(g));
        if (!idle) continue;
        const int sib = s->pcie_pair[g];
        if (sib != g && (taken[sib] || link_busy(sib))) continue;
        taken[g] = 1;
        if (n < cap) helpers[n] = g;
        ++n;
    }
    return n;
}

}  // extern "C"

// =====================================================================================
// Request handling around a swap: what the controller does with every router request and
// every executor completion (include/server/controller.hpp:130-262), and the helpers they
// share -- placement :283-294, check_eviction :392-400, send_exec_req :402-418,
// send_load_req :420-427, lock / unlock of the source replica :442-453.  One request per
// GPU at a time; what finds no idle GPU waits in a FIFO and takes the next GPU that
// completes.  Sockets and executor threads are not part of this: every signal the
// reference would send to an executor, and every acknowledgement it would send to the
// router, goes to a callback, in the order the reference sends them.
#include <deque>

namespace {
constexpr int kRunColdStart = 5;                                                      // controller.hpp:24
constexpr int kSigNotify = 0, kSigStartup = 1, kSigExecute = 2, kSigUnload = 3, kSigLoad = 4;  // utils.hpp:70-74
constexpr int kReqExecuteAfterLoad = 0, kReqExecute = 1, kReqLoad = 2, kReqUnload = 3;         // proto/signal.proto
constexpr int kAckOk = 0;

inline int level_to_status(int level) {   // model_level_to_exec_status (:26-33)
    return (level >= 0 && level <= 2) ? level + kRunPcieLight : kRunPcieMedian;
}

bool parse_int(const char* text, int* out) {
    char* end = nullptr;
    long v = strtol(text, &end, 10);
    if (end == text) return false;
    *out = (int)v;
    return true;
}
}  // namespace

struct tsw_controller {
    int n = 0;
    tsw_scheduler* sched = nullptr;   // executor_status_[i].status_, model_level_map_, schedule_func_
    tsw_evictor* ev = nullptr;
    std::vector<std::string> running;                        // executor_status_[i].function_
    std::map<int, std::pair<int, std::string>> demand;       // executor_gpu_demand_: dst -> (src, func)
    std::deque<std::pair<std::string, bool>> waiting;        // req_queue_: (func, is a cold start)
    int cur_id = 0;
    tsw_signal_fn on_signal = nullptr;
    tsw_ack_fn on_ack = nullptr;
    void* user = nullptr;

    void send(const std::string& func, int gpu, int signal) {
        if (on_signal) on_signal(user, gpu, signal, func.c_str());
    }
    void ack(int gpu) {
        if (on_ack) on_ack(user, kAckOk, gpu);
    }
    int level_of(const std::string& func) {    // model_level_map_[func]: unknown functions read as level 0
        auto it = sched->level.find(func);
        return it == sched->level.end() ? 0 : it->second;
    }
    int placement() {                           // :283-294 with naive() :271-281
        if (sched->status[cur_id] == kAvail) {
            const int g = cur_id;
            cur_id = (cur_id + 1) % n;
            return g;
        }
        for (int i = 0; i < n; ++i)
            if (sched->status[i] == kAvail) return i;
        return -1;
    }
    // A model at or above the limit can never be made room for (`>=`, evictor.hpp:65,85,211);
    // any other refusal by the eviction policy is pins held by GPUs that are still copying.
    bool can_ever_fit(const std::string& func) const { return tsw_repo_total_size(func.c_str()) < ev->budget; }
    int check_eviction(int gpu, const std::string& func, bool must_add = false) {   // :392-400
        std::vector<std::string> victims;
        const int rc = evictor_check_and_add(ev, gpu, func, tsw_repo_total_size(func.c_str()), level_of(func), &victims, -1, must_add);
        if (rc < 0) return rc;
        for (auto& v : victims) {
            tsw_repo_remove_model_info(v.c_str(), gpu);
            send(v, gpu, kSigUnload);
        }
        return TSW_OK;
    }
    void send_exec(const std::string& func, int gpu, int status) {   // :402-418
        if (status == kRunColdStart) {
            for (int i = 0; i < n; ++i) {
                if (i == gpu) {
                    sched->status[i] = kRunColdStart;
                    running[i] = func;
                    send(func, i, kSigStartup);
                } else {
                    send(func, i, kSigNotify);
                }
            }
        } else {
            sched->status[gpu] = status;
            running[gpu] = func;
            send(func, gpu, kSigExecute);
        }
    }
    int send_load(const std::string& func, int dst, int src) {       // :420-427
        bool pinned = false;
        if (src >= 0) {                                               // lock_src_func :442-445
            pinned = demand.insert({dst, {src, func}}).second;
            tsw_evictor_lock(ev, src, func.c_str());
        }
        const int rc = check_eviction(dst, func);
        if (rc != TSW_OK) {                                           // nothing was evicted, nothing sent: undo the pin
            if (src >= 0) tsw_evictor_unlock(ev, src, func.c_str());
            if (pinned) demand.erase(dst);
            return rc;
        }
        send(func, dst, kSigLoad + 1 + src);
        return TSW_OK;
    }
    void unlock_src(int dst) {                                        // :447-453
        auto it = demand.find(dst);
        if (it == demand.end()) return;
        tsw_evictor_unlock(ev, it->second.first, it->second.second.c_str());
        demand.erase(it);
    }
};

extern "C" {

int tsw_ctrl_create(int gpu_count, uint64_t mem_limit_bytes, const char* schedule_policy, const char* evict_policy,
                    const int* pcie_pairs, const int* nvlink, tsw_signal_fn on_signal, tsw_ack_fn on_ack, void* user,
                    tsw_controller** out) {
    if (!out || gpu_count <= 0) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    std::unique_ptr<tsw_controller> c(new tsw_controller());
    c->n = gpu_count;
    int rc = tsw_sched_create(gpu_count, schedule_policy, pcie_pairs, nvlink, &c->sched);
    if (rc != TSW_OK) return rc;
    rc = tsw_evictor_create(evict_policy, gpu_count, mem_limit_bytes, &c->ev);
    if (rc != TSW_OK) {
        tsw_sched_destroy(c->sched);
        return rc;
    }
    c->running.assign(gpu_count, std::string());
    c->on_signal = on_signal;
    c->on_ack = on_ack;
    c->user = user;
    *out = c.release();
    return TSW_OK;
}

int tsw_ctrl_destroy(tsw_controller* c) {
    if (!c) return TSW_OK;
    tsw_sched_destroy(c->sched);
    tsw_evictor_destroy(c->ev);
    delete c;
    return TSW_OK;
}

int tsw_ctrl_request(tsw_controller* c, int type, const char* func_c, const char* payload) {
    if (!c || !func_c) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    const std::string func(func_c);
    const bool has_payload = payload && payload[0];
    int hint = 0;
    const bool reads_payload = type == kReqExecuteAfterLoad || type == kReqExecute || type == kReqUnload;
    if (has_payload && reads_payload && !parse_int(payload, &hint)) return tsw::fail(TSW_ERR_INVALID, "request payload is not a number");

    if (type == kReqExecuteAfterLoad) {                               // :141-162
        int level = kLevelMedian;
        if (has_payload && hint >= 0 && hint <= 2) level = hint;
        c->sched->level[func] = level;
        c->ev->level[func] = level;   // the eviction policy reads the same level map (:393)
        const int gpu = c->placement();
        if (gpu == -1) {
            c->waiting.push_back({func, true});
        } else {
            c->send_exec(func, gpu, kRunColdStart);
            c->ack(gpu);
        }
        return TSW_OK;
    }
    if (type == kReqExecute) {                                        // :163-185
        if (has_payload) {                                            // the router names the GPU
            if (hint < 0 || hint >= c->n) return tsw::fail(TSW_ERR_INVALID, "GPU hint out of range");
            const int rc = c->send_load(func, hint, -1);
            if (rc != TSW_OK) return rc;
            c->send_exec(func, hint, level_to_status(c->level_of(func)));
            c->ack(hint);
            return TSW_OK;
        }
        int gpu, src, status;
        int rc = tsw_sched_decide(c->sched, func_c, &gpu, &src, &status);
        if (rc != TSW_OK) return rc;
        if (gpu == -1) {
            c->waiting.push_back({func, false});
            return TSW_OK;
        }
        rc = c->send_load(func, gpu, src);
        if (rc == TSW_ERR_STATE && c->can_ever_fit(func)) {           // pinned replicas in the way: wait for a completion
            c->waiting.push_back({func, false});
            return TSW_OK;
        }
        if (rc != TSW_OK) return rc;
        c->send_exec(func, gpu, status);
        c->ack(gpu);
        return TSW_OK;
    }
    if (type == kReqUnload) {                                         // :186-206
        int homes[256];
        int nh = tsw_repo_active_devices(func_c, homes, 256);
        if (nh > 256) nh = 256;
        for (int i = 0; i < nh; ++i) {
            const int g = homes[i];
            if (g < 0 || g >= c->n) continue;
            if (has_payload && g != hint) continue;
            tsw_evictor_force_evict(c->ev, g, func_c);
            tsw_repo_remove_model_info(func_c, g);
            c->send(func, g, kSigUnload);
        }
        c->ack(-1);
        return TSW_OK;
    }
    if (type == kReqLoad) {                                           // :207-214: a replica on every GPU
        for (int i = 0; i < c->n; ++i) {
            const int rc = c->send_load(func, i, -1);
            if (rc != TSW_OK) return rc;
            tsw_repo_add_model_info(func_c, i);
        }
        c->ack(-1);
        return TSW_OK;
    }
    return TSW_OK;   // other request types are not the controller's (:139-214 has no branch for them)
}

int tsw_ctrl_complete(tsw_controller* c, int executor) {              // :217-262
    if (!c || executor < 0 || executor >= c->n) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    const int st = c->sched->status[executor];
    const std::string done = c->running[executor];
    int rc = TSW_OK;
    if (st == kRunColdStart) {            // a cold start enters the cache here, and may push others out
        tsw_repo_add_model_info(done.c_str(), executor);
        rc = c->check_eviction(executor, done, /*must_add=*/true);   // it is on the GPU already
    } else if (st > kAvail && st < kRunColdStart) {
        tsw_repo_add_model_info(done.c_str(), executor);
    }
    c->unlock_src(executor);
    c->sched->status[executor] = kAvail;
    if (rc != TSW_OK) return rc;

    if (!c->waiting.empty()) {
        const std::pair<std::string, bool> next = c->waiting.front();
        c->waiting.pop_front();
        if (next.second) {
            c->send_exec(next.first, executor, kRunColdStart);
        } else {
            int gpu, src, status;
            rc = tsw_sched_decide(c->sched, next.first.c_str(), &gpu, &src, &status);
            if (rc != TSW_OK) return rc;
            if (gpu != executor) {        // the freed GPU is the only option: load from the host store
                src = -1;
                status = level_to_status(c->level_of(next.first));
            }
            rc = c->send_load(next.first, executor, src);
            if (rc == TSW_ERR_STATE && c->can_ever_fit(next.first)) {   // pins in the way: it keeps its place in the queue
                c->waiting.push_front(next);
                return TSW_OK;
            }
            if (rc != TSW_OK) return rc;
            c->send_exec(next.first, executor, status);
        }
        c->ack(executor);
    }
    return TSW_OK;
}

int tsw_ctrl_executor_status(tsw_controller* c, int gpu, int* status, char* func, int cap) {
    if (!c || gpu < 0 || gpu >= c->n) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    if (status) *status = c->sched->status[gpu];
    if (func && cap > 0) {
        const std::string& f = c->running[gpu];
        if ((int)f.size() + 1 > cap) return tsw::fail(TSW_ERR_BUFFER, "function name buffer too small");
        memcpy(func, f.c_str(), f.size() + 1);
    }
    return TSW_OK;
}

int tsw_ctrl_helpers(tsw_controller* c, int dst, int include_running, int* helpers, int cap) {
    if (!c) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    return tsw_sched_helpers(c->sched, dst, include_running, helpers, cap);
}

int tsw_ctrl_queue_depth(tsw_controller* c) {
    if (!c) return tsw::fail(TSW_ERR_INVALID, "bad controller arguments");
    return (int)c->waiting.size();
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
