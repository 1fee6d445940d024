// Swap scheduler: which GPU runs a request, and where its weights come from; and the machine
// topology it reads (C ABI).
//
// The decision functions of the reference's controller (include/server/controller.hpp:
// random_schedule :296-318, interference_aware_schedule :321-389, model_level_to_exec_status
// :26-33) for any number of GPUs.  The reference hard-codes a 4-GPU box (pcie_pairs_ and
// nvlink_topology_, :116-118); here both tables are inputs.  With no tables given the
// defaults describe an NVSwitch machine: every peer is a "fast" NVLink neighbour, and GPU i
// shares its PCIe uplink with GPU i^1.

#include "policy_internal.hpp"

using namespace tsw_policy;

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
