// TEST INFRASTRUCTURE ONLY.  Shadow of the reference's common/include/socket_helper.hpp so that
// include/server/controller.hpp compiles where it lies without ZeroMQ.  The controller's loop
// (controller.hpp:125-264) polls this stand-in: a hook set by the harness hands it the next
// scripted router request (or injects an executor completion and reports "no request"), and
// ends the otherwise endless loop by throwing Stop when the script is used up.  What the
// controller sends back to the router is appended to the trace.
#ifndef TORPOR_REF_SHIM_SOCKET_HELPER_HPP_
#define TORPOR_REF_SHIM_SOCKET_HELPER_HPP_

#include "types.hpp"

#include <functional>

#define ZMQ_REP 4
#define ZMQ_POLLIN 1

namespace zmq {
struct context_t {};
struct socket_t {
    socket_t() {}
    socket_t(context_t&, int) {}
    void bind(const string&) {}
    operator void*() { return this; }
};
struct pollitem_t {
    void* socket;
    int fd;
    short events;
    short revents;
};
}  // namespace zmq

namespace torpor_ref_script {
struct Stop {};
struct State {
    std::function<bool(string* request)> next;   // true: a request is waiting; may throw Stop
    vector<string> trace;                        // "S gpu signal func" and "A ack resp" lines
};
inline State& state() {
    static State s;
    return s;
}
}  // namespace torpor_ref_script

struct ZmqUtilShim {
    int poll(long, vector<zmq::pollitem_t>* items) {
        auto& st = torpor_ref_script::state();
        (*items)[0].revents = 0;
        if (st.next && st.next(&pending_)) (*items)[0].revents = ZMQ_POLLIN;
        return 0;
    }
    string recv_string(zmq::socket_t*) { return pending_; }
    void send_string(const string& ack, zmq::socket_t*) { torpor_ref_script::state().trace.push_back("A " + ack); }
    string pending_;
};
static ZmqUtilShim zmq_util_shim;
static ZmqUtilShim* kZmqUtil = &zmq_util_shim;

inline string get_signal_addr(int id) { return "ipc:///cuda/signal_" + std::to_string(id); }
inline string get_client_addr(int id) { return "ipc:///cuda/client_" + std::to_string(id); }

#endif
