// The reference's own controller (include/server/controller.hpp, unmodified, compiled where it
// lies) running on top of the drop-in adapter: its ModelRepo and Evictor are the headers of
// torpor_b200/adapter over libtorpor_swap.so, its MemoryManager the adapter class on a plan-only
// engine.  Sockets and executors are the stand-ins of oracle/ref_shim_ctrl (one scripted event per
// turn of Controller::start; signals and acknowledgements recorded).  tests/test_adapter.py drives
// this program over a pipe with the event streams of tests/controller_cases.py and holds the
// traces to the recordings made from the reference alone.
//
// The adapter headers are included FIRST: they carry the reference's include guards, so the
// `#include "model_repo.hpp"` / `"evictor.hpp"` lines inside controller.hpp (which the compiler
// would resolve to the neighbouring originals, whatever the include path says) contribute nothing.
#include "cuda_common.hpp"
#include "utils.hpp"
#include "safe_ptr.hpp"
#include "spdlog/spdlog.h"
#include "spdlog/sinks/null_sink.h"

#include "memory_manager.hpp"   // torpor_b200/adapter (includes its model_repo.hpp)
#include "evictor.hpp"          // torpor_b200/adapter
#include "cuda_server.hpp"      // oracle/ref_shim_ctrl: the executor stand-in
#define INCLUDE_CUDA_SERVER_HPP_
#define private public
#include "controller.hpp"       // the reference's own
#undef private

#include <iostream>
#include <sstream>

static void run_one_event(server::Controller& c, const std::string* request, int executor) {
    auto& st = torpor_ref_script::state();
    st.trace.clear();
    int polls = 0;
    st.next = [&](string* r) -> bool {
        if (polls++ > 0) throw torpor_ref_script::Stop();
        if (request) { *r = *request; return true; }
        server::controller_sync_queue->push(executor);
        return false;
    };
    try {
        c.start();
    } catch (const torpor_ref_script::Stop&) {
    }
    st.next = nullptr;
    for (auto& t : c.thread_vec_) if (t.joinable()) t.join();
    c.thread_vec_.clear();
}

int main() {
    using namespace server;
    using namespace server::manager;
    std::streambuf* console = std::cout.rdbuf();
    std::ostringstream chatter;                      // the controller prints on every event
    auto quiet = std::make_shared<spdlog::logger>("probe", std::make_shared<spdlog::sinks::null_sink_mt>());
    setenv("TORPOR_SWAP_DEVICE", "-1", 1);
    MemoryManager mm(0);
    mm.set_logger(quiet);
    mm.set_server_id(0);
    std::cout.rdbuf(chatter.rdbuf());
    mm.start_trans_thread(4);
    std::cout.rdbuf(console);
    if (!mm.engine()) return 2;

    zmq::context_t ctx;
    std::unique_ptr<Controller> ctrl;
    std::string line;
    while (std::getline(std::cin, line)) {
        std::istringstream in(line);
        std::string op;
        in >> op;
        std::cout.rdbuf(chatter.rdbuf());
        std::vector<std::string> answer;
        if (op == "T") {                             // T <func>: cold start begins
            std::string f; in >> f;
            mm.set_track_model_memory(f);
        } else if (op == "M") {                      // M <func> <bytes> <is_model>
            std::string f; size_t bytes; int is_model; in >> f >> bytes >> is_model;
            if (!mm.cudaMallocBackend(bytes, is_model != 0, f)) answer.push_back("E malloc");
        } else if (op == "U") {                      // U <func>: cold start ends
            std::string f; in >> f;
            mm.unset_track_model_memory(f);
        } else if (op == "N") {                      // N <limit GiB> <SCHEDULE_POLICY> <EVICT_POLICY>
            int gib; std::string sp, ep; in >> gib >> sp >> ep;
            setenv("MEM_LIMIT_IN_GB", std::to_string(gib).c_str(), 1);
            if (sp == "RAND") setenv("SCHEDULE_POLICY", "RAND", 1); else unsetenv("SCHEDULE_POLICY");
            if (ep == "LRU") setenv("EVICT_POLICY", "LRU", 1); else unsetenv("EVICT_POLICY");
            torpor_ref_fake::device_count() = 4;
            srand(1);
            ctrl.reset(new Controller(quiet, &ctx));
        } else if (op == "R" && ctrl) {              // R <type> <func> [payload]
            std::string type, f, payload; in >> type >> f >> payload;
            const std::string req = type + " " + f + " " + payload;
            run_one_event(*ctrl, &req, -1);
            answer = torpor_ref_script::state().trace;
        } else if (op == "C" && ctrl) {              // C <executor>
            int g; in >> g;
            run_one_event(*ctrl, nullptr, g);
            answer = torpor_ref_script::state().trace;
        } else if (op == "Q") {
            std::cout.rdbuf(console);
            break;
        } else {
            answer.push_back("E unknown command");
        }
        std::cout.rdbuf(console);
        chatter.str("");
        for (auto& a : answer) std::cout << a << "\n";
        std::cout << "." << std::endl;
    }
    std::cout.rdbuf(console);
    if (ctrl) ctrl.release();                        // its executor threads were joined; leave the rest to exit
    mm.destroy_trans_thread();
    return 0;
}
