// TEST INFRASTRUCTURE ONLY.  Shadow of the reference's include/server/cuda_server.hpp for
// compiling include/server/controller.hpp where it lies: the executor is reduced to the two
// members the controller touches.  Signals the controller sends are recorded, not executed.
#ifndef TORPOR_REF_SHIM_CUDA_SERVER_HPP_
#define TORPOR_REF_SHIM_CUDA_SERVER_HPP_

#include "cuda_common.hpp"
#include "utils.hpp"
#include "safe_ptr.hpp"
#include "socket_helper.hpp"

namespace server {

static sf::safe_ptr<queue<int>> controller_sync_queue;

class CUDAExecutor {
public:
    CUDAExecutor(int id, size_t, zmq::context_t*) : id_(id) {}
    void start() {}
    void sig_exec_from_controller(int signal, string& func) {
        torpor_ref_script::state().trace.push_back("S " + std::to_string(id_) + " " + std::to_string(signal) + " " + func);
    }
private:
    int id_;
};

}  // namespace server

#endif
