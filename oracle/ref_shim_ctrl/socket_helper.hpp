// TEST INFRASTRUCTURE ONLY.  Shadow of the reference's common/include/socket_helper.hpp so that
// include/server/controller.hpp compiles where it lies without ZeroMQ: the controller's socket
// calls become no-ops; only its decision functions are exercised by the harness.
#ifndef TORPOR_REF_SHIM_SOCKET_HELPER_HPP_
#define TORPOR_REF_SHIM_SOCKET_HELPER_HPP_

#include "types.hpp"

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

struct ZmqUtilShim {
    int poll(long, vector<zmq::pollitem_t>*) { return 0; }
    string recv_string(zmq::socket_t*) { return string(); }
    void send_string(const string&, zmq::socket_t*) {}
};
static ZmqUtilShim zmq_util_shim;
static ZmqUtilShim* kZmqUtil = &zmq_util_shim;

inline string get_signal_addr(int id) { return "ipc:///cuda/signal_" + std::to_string(id); }
inline string get_client_addr(int id) { return "ipc:///cuda/client_" + std::to_string(id); }

#endif
