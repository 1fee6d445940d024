// The reference's own executor (include/server/cuda_server.hpp, unmodified, compiled where it lies)
// running on top of the drop-in adapter: its `mem_manager_` member is the MemoryManager of
// torpor_b200/adapter over libtorpor_swap.so, on a plan-only engine.  Message classes are the
// stand-ins generated from the reference's .proto files, sockets those of oracle/ref_shim_exec, cuDNN
// and cuBLAS stubs.  The executor's loop runs on a thread; tests/test_adapter.py drives this program
// over a pipe -- controller signals, serialised QueryLists -- with the streams it also gives the
// reference's executor over the reference's own manager, and holds responses, launch arguments and
// tables of the two to each other.
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

#include <deque>
#include <iostream>
#include <sstream>
#include <thread>

map<string, const void*>& lookup() {
    static map<string, const void*> table;
    return table;
}
map<string, KernelAccessLoc>& kernel_model_access_loc() {
    static map<string, KernelAccessLoc> table;
    return table;
}

namespace {
struct Launch { std::string kernel; std::vector<std::string> args; };
std::mutex g_mu;
std::deque<std::vector<size_t>> g_sizes;
std::vector<Launch> g_launches;

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

namespace torpor_ref_fake {
void record_launch(const void* func, void** args) {
    std::lock_guard<std::mutex> g(g_mu);
    Launch l;
    for (auto& kv : lookup()) if (kv.second == func) l.kernel = kv.first;
    if (!g_sizes.empty()) {
        auto sizes = g_sizes.front();
        g_sizes.pop_front();
        for (size_t i = 0; i < sizes.size(); ++i) l.args.emplace_back((const char*)args[i], sizes[i]);
    }
    g_launches.push_back(l);
}
}  // namespace torpor_ref_fake

int main() {
    using namespace server;
    std::streambuf* console = std::cout.rdbuf();
    std::ostringstream chatter;
    setenv("TORPOR_SWAP_DEVICE", "-1", 1);
    torpor_ref_fake::device_count() = 1;
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
    static char anchors[64];
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream in(line);
        std::string op;
        in >> op;
        std::vector<std::string> answer;
        if (op == "K") {                                  // K <kernel name>
            std::string k; in >> k;
            if (!lookup().count(k)) lookup()[k] = &anchors[lookup().size()];
        } else if (op == "S") {                           // S <signal> <func>
            int sig; std::string f; in >> sig >> f;
            ex->sig_exec_from_controller(sig, f);
        } else if (op == "Q") {                           // Q <hex of a serialised QueryList>
            std::string h; in >> h;
            const std::string msg = unhex(h);
            {
                QueryList ql;
                ql.ParseFromString(msg);
                std::lock_guard<std::mutex> g(g_mu);
                for (auto& q : ql.queries()) {
                    if (q.type() != QueryType::cudaLaunchKernel) continue;
                    cudaLaunchKernelQuery lq;
                    lq.ParseFromString(q.query());
                    if (!lookup().count(lq.function())) continue;
                    std::vector<size_t> sizes;
                    for (int i = 0; i < lq.args_size(); ++i) sizes.push_back(lq.args(i).length());
                    g_sizes.push_back(sizes);
                }
            }
            std::vector<std::string> sent;
            {
                std::unique_lock<std::mutex> lk(channel.mu);
                channel.inbox.push_back(msg);
                channel.cv.notify_all();
                channel.cv.wait(lk, [&] { return channel.inbox.empty() && !channel.busy; });
                sent.swap(channel.sent);
            }
            for (auto& s : sent) answer.push_back("R " + hex(s));
        } else if (op == "L") {                           // launches since the last L
            std::lock_guard<std::mutex> g(g_mu);
            for (auto& l : g_launches) {
                std::string t = "L " + l.kernel;
                for (auto& a : l.args) t += " " + hex(a);
                answer.push_back(t);
            }
            g_launches.clear();
        } else if (op == "C") {                           // executor ids on controller_sync_queue
            while (!controller_sync_queue->empty()) {
                answer.push_back("C " + std::to_string(controller_sync_queue->front()));
                controller_sync_queue->pop();
            }
        } else if (op == "B" || op == "P") {              // B/P <func>: block / parameter table of the engine
            std::string f; in >> f;
            tsw_engine* e = ex->mem_manager_.engine();
            const int width = op == "B" ? 6 : 7;
            int n = op == "B" ? tsw_dump_blocks(e, f.c_str(), 0, nullptr, 0) : tsw_dump_params(e, f.c_str(), 0, nullptr, 0);
            std::vector<uint64_t> rows((size_t)std::max(n, 1) * width);
            if (op == "B") tsw_dump_blocks(e, f.c_str(), 0, rows.data(), n); else tsw_dump_params(e, f.c_str(), 0, rows.data(), n);
            for (int r = 0; r < n; ++r) {
                std::string t = "T";
                for (int c = 0; c < width; ++c) t += " " + std::to_string(rows[(size_t)r * width + c]);
                answer.push_back(t);
            }
        } else if (op == "A") {                           // A <func>: check_model_alloc_status
            std::string f; in >> f;
            answer.push_back(std::string("A ") + (ex->mem_manager_.check_model_alloc_status(f) ? "1" : "0"));
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
    ex->mem_manager_.destroy_trans_thread();
    return 0;                                            // the executor object is left to process exit
}
