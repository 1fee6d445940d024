// Drop-in for include/server/evictor.hpp: Evictor, LRUEvictor and InterferenceAwareEvictor
// with the reference's constructor and virtual interface (evictor.hpp:14-26), decisions
// made by libtorpor_swap.so.  When nothing can be evicted the reference spins
// (evictor.hpp:84-95,211-224); here check_and_add prints the reason and returns no victims.
#ifndef INCLUDE_EVICTOR_HPP_
#define INCLUDE_EVICTOR_HPP_

#include <algorithm>
#include <iostream>
#include <list>
#include "utils.hpp"
#include "torpor_swap.h"

namespace server {

const int ModelLevel_Light = 0;
const int ModelLevel_Median = 1;
const int ModelLevel_Heavy = 2;

class Evictor {
public:
    Evictor(int gpu_count, size_t budget) : gpu_count_(gpu_count), budget_(budget) {}
    virtual ~Evictor() {
        if (impl_) tsw_evictor_destroy(impl_);
    }

    virtual vector<string> check_and_add(int gpu_idx, string& func, size_t sz, map<string, int>& model_level_map) {
        vector<string> out;
        std::vector<char> buf(1 << 16);
        int n = tsw_evictor_check_and_add(impl_, gpu_idx, func.c_str(), sz, model_level_map[func], buf.data(), (int)buf.size());
        if (n < 0) {
            std::cout << "Controller -- evictor: " << tsw_last_error() << std::endl;
            return out;
        }
        string joined(buf.data());
        size_t pos = 0;
        while (n > 0 && pos <= joined.size()) {
            size_t nl = joined.find('\n', pos);
            out.push_back(joined.substr(pos, nl == string::npos ? string::npos : nl - pos));
            if (nl == string::npos) break;
            pos = nl + 1;
        }
        return out;
    }
    virtual void force_evict(int gpu_idx, string& func) { tsw_evictor_force_evict(impl_, gpu_idx, func.c_str()); }
    virtual void lock(int gpu_idx, string& func) { tsw_evictor_lock(impl_, gpu_idx, func.c_str()); }
    virtual void unlock(int gpu_idx, string& func) { tsw_evictor_unlock(impl_, gpu_idx, func.c_str()); }

protected:
    void make(const char* kind) { tsw_evictor_create(kind, gpu_count_, budget_, &impl_); }
    int gpu_count_;
    size_t budget_;
    tsw_evictor* impl_ = nullptr;
};

class InterferenceAwareEvictor : public Evictor {
public:
    InterferenceAwareEvictor(int gpu_count, size_t budget) : Evictor(gpu_count, budget) { make("IA"); }
};

class LRUEvictor : public Evictor {
public:
    LRUEvictor(int gpu_count, size_t budget) : Evictor(gpu_count, budget) { make("LRU"); }
};

}  // namespace server

#endif  // INCLUDE_EVICTOR_HPP_
