// Drop-in for include/server/model_repo.hpp when the swap path is served by
// libtorpor_swap.so.  The heavy tables (blocks, parameters, host copies, per-GPU
// placement) live inside the library; this singleton keeps exactly the members the
// controller reads and writes (include/server/controller.hpp:191-203,212,225,230,
// 308-344,393-396) and forwards the two status calls so that the library knows which
// replicas are healthy sources for a GPU-to-GPU swap (memory_manager.hpp:213-224).
#ifndef INCLUDE_MODEL_REPO_HPP_
#define INCLUDE_MODEL_REPO_HPP_

#include "cuda_common.hpp"
#include "utils.hpp"
#include "torpor_swap.h"

namespace server {
namespace manager {

const int ModelStatus_Full = 0;
const int ModelStatus_Incomplete = 1;
const int ModelStatus_Partial = 2;
const int ModelStatus_NoData = 3;

struct HostModelInfo {
    int status_ = ModelStatus_Incomplete;
    size_t total_size_ = 0;
};

struct DeviceModelInfo {
    int status_ = ModelStatus_Incomplete;
};

class ModelRepo {
public:
    static ModelRepo& getInstance() {
        static ModelRepo repo;
        return repo;
    }

    void init_device_info(int device_id) { device_model_info_map_[device_id] = {}; }

    void add_model_info(string& function, int gpu_id) {
        device_model_info_map_[gpu_id][function].status_ = ModelStatus_Full;
        model_active_device_map_[function].insert(gpu_id);
        tsw_repo_add_model_info(function.c_str(), gpu_id);
    }

    void remove_model_info(string& function, int gpu_id) {
        device_model_info_map_[gpu_id][function].status_ = ModelStatus_NoData;
        model_active_device_map_[function].erase(gpu_id);
        tsw_repo_remove_model_info(function.c_str(), gpu_id);
    }

    void start_model_load(string& function) { model_host_info_map_[function].status_ = ModelStatus_Incomplete; }
    void complete_model_load(string& function) { model_host_info_map_[function].status_ = ModelStatus_Full; }

private:
    ModelRepo() {}

public:
    map<string, HostModelInfo> model_host_info_map_;
    map<int, map<string, DeviceModelInfo>> device_model_info_map_;
    map<string, set<int>> model_active_device_map_;
};

}  // namespace manager
}  // namespace server

#endif  // INCLUDE_MODEL_REPO_HPP_
