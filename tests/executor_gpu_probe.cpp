// The reference's own executor (include/server/cuda_server.hpp, unmodified, compiled where it lies)
// on a real GPU, with the drop-in adapter as its `mem_manager_`: serialised QueryLists and controller
// signals go in over a pipe (tests/test_gpu_adapter.py), its loop dispatches them as in service --
// cudaMalloc / cudaMemcpy services through the adapter into libtorpor_swap.so, the swap signal into
// place_kernel, cudaLaunchKernelService rewriting pointer words and launching real kernels
// (tests/wire_kernels.cu, linked in) on the executor's own stream -- and its serialised responses
// come back.  The CUDA runtime is the real one; message classes are the stand-ins generated from
// the reference's .proto files, sockets those of oracle/ref_shim_exec, cuDNN and cuBLAS stubs.
//
// The adapter header comes FIRST: it carries the reference's include guard, so the
// `#include "memory_manager.hpp"` inside cuda_server.hpp adds nothing.
#include "cuda_common.hpp"
#include "utils.hpp"
#include "safe_ptr.hpp"
#include "spdlog/spdlog.h"
#include "spdlog/sinks/null_sink.h"

#include "memory_manager.hpp"   // torpor_b200/adapter

namespace spdlog {
inline std::shared_ptr<logger> torpor_fileless_logger(const std::string& name, const std::string&, bool = false) {
    return std::make_shared<logger>(name, std::make_shared<sinks::null_sink_mt>());
}
}  // namespace spdlog
#define basic_logger_mt torpor_fileless_logger   // the executor's constructor opens a log file (cuda_server.hpp:57-59)
#define private public
#include "cuda_server.hpp"      // the reference's own
#undef private
#undef basic_logger_mt

#include <iostream>
#include <sstream>
#include <thread>

// host-side handles of the kernels in tests/wire_kernels.cu (the generated table of src/server/kernel_lookup.cpp
// holds such handles for the kernels of the client's libraries)
extern "C" void wire_saxpy(const float*, const float*, float*, unsigned long long, float);
struct WirePair;
extern "C" void wire_scale_pair(WirePair, float);

map<string, const void*>& lookup() {
    static map<string, const void*> table;
    return table;
}
map<string, KernelAccessLoc>& kernel_model_access_loc() {
    static map<string, KernelAccessLoc> table;
    return table;
}

namespace {
std::string hex(const std::string& s) {
    static const char* d = "0123456789abcdef";
    std::string o;
    for (unsigned char c : s) { o += d[c >> 4]; o += d[c & 15]; }
    return o.empty() ? "-" : o;
}
std::string unhex(const std::string& h) {
    std::string o;
    if (h == "-") return o;
    for (size_t i = 0; i + 1 < h.size(); i += 2) o += (char)std::stoi(h.substr(i, 2), nullptr, 16);
    return o;
}
}  // namespace

int main() {
    using namespace server;
    std::streambuf* console = std::cout.rdbuf();
    std::ostringstream chatter;
    zmq::context_t ctx;
    std::cout.rdbuf(chatter.rdbuf());
    auto* ex = new CUDAExecutor(0, 0, &ctx);
    auto& channel = torpor_ref_exec::channel_of((void*)&ex->srv_pull_handler_);
    std::thread loop([ex] {
        try {
            ex->start();
        } catch (const torpor_ref_exec::Stop&) {
        }
    });
    {
        std::unique_lock<std::mutex> lk(channel.mu);
        channel.cv.wait(lk, [&] { return channel.polls > 0; });
    }
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream in(line);
        std::string op;
        in >> op;
        std::vector<std::string> answer;
        if (op == "K") {                                  // K <kernel name>: enter it in the executor's kernel table
            std::string k; in >> k;
            if (k == "wire_saxpy") lookup()[k] = (const void*)&wire_saxpy;
            else if (k == "wire_scale_pair") lookup()[k] = (const void*)&wire_scale_pair;
            else answer.push_back("E unknown kernel");
        } else if (op == "S") {                           // S <signal> <func>
            int sig; std::string f; in >> sig >> f;
            ex->sig_exec_from_controller(sig, f);
        } else if (op == "Q") {                           // Q <hex of a serialised QueryList>
            std::string h; in >> h;
            std::vector<std::string> sent;
            {
                std::unique_lock<std::mutex> lk(channel.mu);
                channel.inbox.push_back(unhex(h));
                channel.cv.notify_all();
                channel.cv.wait(lk, [&] { return channel.inbox.empty() && !channel.busy; });
                sent.swap(channel.sent);
            }
            for (auto& s : sent) answer.push_back("R " + hex(s));
        } else if (op == "C") {                           // executor ids on controller_sync_queue
            while (!controller_sync_queue->empty()) {
                answer.push_back("C " + std::to_string(controller_sync_queue->front()));
                controller_sync_queue->pop();
            }
        } else if (op == "G") {                           // G <func> <client pointer>: where the parameter is now
            std::string f; unsigned long long p; in >> f >> p;
            answer.push_back("G " + std::to_string((unsigned long long)ex->mem_manager_.get_cuda_addr(f, (void*)p)));
        } else if (op == "N") {                           // kernel launches and bytes moved by the engine so far
            uint64_t launches = 0, bytes = 0, ns = 0;
            tsw_stats(ex->mem_manager_.engine(), &launches, &bytes, &ns);
            answer.push_back("N " + std::to_string(launches) + " " + std::to_string(bytes));
        } else if (op == "X") {
            break;
        } else {
            answer.push_back("E unknown command");
        }
        std::cout.rdbuf(console);
        for (auto& a : answer) std::cout << a << "\n";
        std::cout << "." << std::endl;
        std::cout.rdbuf(chatter.rdbuf());
        chatter.str("");
    }
    {
        std::lock_guard<std::mutex> g(channel.mu);
        channel.stop = true;
        channel.cv.notify_all();
    }
    loop.join();
    std::cout.rdbuf(console);
    cudaDeviceSynchronize();
    ex->mem_manager_.destroy_trans_thread();
    return 0;                                            // the executor object is left to process exit
}
