// Request handling around a swap (C ABI), over the scheduler and the eviction policy: what the controller does with every router request and
// every executor completion (include/server/controller.hpp:130-262), and the helpers they
// share -- placement :283-294, check_eviction :392-400, send_exec_req :402-418,
// send_load_req :420-427, lock / unlock of the source replica :442-453.  One request per
// GPU at a time; what finds no idle GPU waits in a FIFO and takes the next GPU that
// completes.  Sockets and executor threads are not part of this: every signal the
// reference would send to an executor, and every acknowledgement it would send to the
// router, goes to a callback, in the order the reference sends them.

#include "policy_internal.hpp"

#include <deque>

using namespace tsw_policy;

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
