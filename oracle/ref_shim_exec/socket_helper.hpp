// TEST INFRASTRUCTURE ONLY.  Shadow of the reference's common/include/socket_helper.hpp so that
// include/server/cuda_server.hpp (the executor) compiles where it lies without ZeroMQ.  Every
// executor's loop (cuda_server.hpp:99-262) polls this stand-in: it finds the serialised QueryLists
// the harness has queued for it, and what the executor sends back to its clients is kept, in
// order, for the harness to read.  The loop never ends by itself; it is ended by an exception
// from poll when the harness asks for it.
#ifndef TORPOR_REF_SHIM_EXEC_SOCKET_HELPER_HPP_
#define TORPOR_REF_SHIM_EXEC_SOCKET_HELPER_HPP_

#include "types.hpp"

#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>

#define ZMQ_REP 4
#define ZMQ_PULL 7
#define ZMQ_PUSH 8
#define ZMQ_POLLIN 1

namespace zmq {
struct context_t {};
struct socket_t {
    socket_t() {}
    socket_t(context_t&, int) {}
    void bind(const string&) {}
    void connect(const string&) {}
    operator void*() { return this; }
};
struct pollitem_t {
    void* socket;
    int fd;
    short events;
    short revents;
};
}  // namespace zmq

namespace torpor_ref_exec {
struct Stop {};
struct Channel {                       // one per executor, found by the address of its pull socket
    std::mutex mu;
    std::condition_variable cv;
    std::deque<string> inbox;          // serialised QueryLists not yet received
    std::vector<string> sent;          // serialised responses, in the order they were sent
    bool busy = false;                 // a received QueryList is being worked on
    uint64_t polls = 0;                // times the loop has come to its poll
    bool stop = false;
};
inline std::mutex& registry_mu() { static std::mutex m; return m; }
inline std::map<void*, Channel*>& registry() { static std::map<void*, Channel*> r; return r; }
inline Channel& channel_of(void* pull_socket) {
    std::lock_guard<std::mutex> g(registry_mu());
    Channel*& c = registry()[pull_socket];
    if (!c) c = new Channel();
    return *c;
}
inline Channel*& current() { thread_local Channel* c = nullptr; return c; }
}  // namespace torpor_ref_exec

struct ZmqUtilShim {
    int poll(long, vector<zmq::pollitem_t>* items) {
        using namespace torpor_ref_exec;
        Channel& c = channel_of((*items)[0].socket);
        current() = &c;
        std::unique_lock<std::mutex> lk(c.mu);
        c.busy = false;
        c.polls++;
        c.cv.notify_all();
        if (c.stop) throw Stop();
        if (c.inbox.empty()) c.cv.wait_for(lk, std::chrono::milliseconds(1));
        if (c.stop) throw Stop();
        (*items)[0].revents = c.inbox.empty() ? 0 : ZMQ_POLLIN;
        return 0;
    }
    string recv_string(zmq::socket_t* s) {
        using namespace torpor_ref_exec;
        Channel& c = channel_of((void*)s);
        std::lock_guard<std::mutex> g(c.mu);
        string m = c.inbox.front();
        c.inbox.pop_front();
        c.busy = true;
        return m;
    }
    void send_string(const string& m, zmq::socket_t*) {
        using namespace torpor_ref_exec;
        if (!current()) return;
        std::lock_guard<std::mutex> g(current()->mu);
        current()->sent.push_back(m);
    }
};
static ZmqUtilShim zmq_util_shim;
static ZmqUtilShim* kZmqUtil = &zmq_util_shim;

inline string get_client_addr(int id) { return "ipc:///cuda/client_" + std::to_string(id); }
inline string get_server_addr(int id) { return "ipc:///cuda/server_" + std::to_string(id); }
inline string get_signal_addr(int id) { return "ipc:///cuda/signal_" + std::to_string(id); }

class Pusher {
public:
    explicit Pusher(zmq::context_t*) {}
    zmq::socket_t& At(const string& addr) { return cache_[addr]; }
    zmq::socket_t& operator[](const string& addr) { return cache_[addr]; }
    void create(const string& addr) { cache_[addr]; }
    void clear() { cache_.clear(); }
private:
    std::map<string, zmq::socket_t> cache_;
};

#endif
