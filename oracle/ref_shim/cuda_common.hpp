// TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
//
// Shadow of the reference's common/include/cuda_common.hpp, placed FIRST on the
// include path when the reference's swap-path headers
// (include/server/{memory_manager,block_manager,model_repo}.hpp) are compiled
// where they lie, unmodified.  The real header pulls in protoc-generated
// cudarpc.pb.h / signal.pb.h (protoc is not available) and cuDNN/cuBLAS; none
// of those types are used by the three swap-path headers, which only need the
// CUDA runtime calls below and the cudaCheck macro
// (common/include/cuda_common.hpp:108-114).
//
// Two variants:
//   -DTORPOR_REF_FAKE_CUDA : a host-memory stand-in for the CUDA runtime with a
//        DETERMINISTIC address space, so that the reference's pointer-keyed
//        hash maps iterate in a reproducible order.  "Device" memory of GPU g
//        is a lazily committed mmap at kCanonBase + g * kCanonStride, handed
//        out by a 2 MiB-aligned bump allocator.
//   (default)               : the real <cuda_runtime.h>; used for the timed
//        reference arm on a GPU machine.
#ifndef TORPOR_REF_SHIM_CUDA_COMMON_HPP_
#define TORPOR_REF_SHIM_CUDA_COMMON_HPP_

#include "types.hpp"

#include <cassert>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <chrono>
#include <thread>
#include <memory>
#include <iostream>
#include <functional>
#include <algorithm>

#ifndef TORPOR_REF_FAKE_CUDA

#include <cuda_runtime.h>
#include <cuda_runtime_api.h>

#else  // ---------------------------------------------------------------- fake

#include <sys/mman.h>
#include <mutex>

typedef int cudaError_t;
static const cudaError_t cudaSuccess = 0;
static const cudaError_t cudaErrorMemoryAllocation = 2;
typedef void* cudaStream_t;
typedef void* cudaEvent_t;
enum cudaMemcpyKind {
    cudaMemcpyHostToHost = 0,
    cudaMemcpyHostToDevice = 1,
    cudaMemcpyDeviceToHost = 2,
    cudaMemcpyDeviceToDevice = 3,
    cudaMemcpyDefault = 4
};
static const unsigned int cudaStreamNonBlocking = 1;
inline int format_as(cudaMemcpyKind k) { return (int)k; }   // how the reference's logger prints it

namespace torpor_ref_fake {

static const uint64_t kCanonBase = 0x600000000000ull;    // canonical device VA of GPU 0
static const uint64_t kCanonStride = 0x010000000000ull;  // 1 TiB of VA per fake GPU
static const uint64_t kAlign = 2ull << 20;
static const int kMaxDev = 16;

struct DevSpace {
    uint64_t mapped_end = 0;  // bytes of VA currently mmap'ed from the base
    uint64_t bump = 0;        // next offset handed out
};

struct World {
    std::mutex mu;
    DevSpace dev[kMaxDev];
};

inline World& world() {
    static World w;
    return w;
}

inline int& cur_device() {
    thread_local int d = 0;
    return d;
}

inline void* dev_alloc(size_t size) {
    World& w = world();
    std::lock_guard<std::mutex> g(w.mu);
    int d = cur_device();
    DevSpace& s = w.dev[d];
    uint64_t base = kCanonBase + (uint64_t)d * kCanonStride;
    uint64_t off = s.bump;
    uint64_t need = (size + kAlign - 1) / kAlign * kAlign;
    if (off + need > kCanonStride) return nullptr;
    if (off + need > s.mapped_end) {
        // grow the mapping in 1 GiB steps; pages are committed only when touched
        uint64_t grow_to = ((off + need) + (1ull << 30) - 1) / (1ull << 30) * (1ull << 30);
        void* want = (void*)(base + s.mapped_end);
        void* got = mmap(want, grow_to - s.mapped_end, PROT_READ | PROT_WRITE,
                         MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED_NOREPLACE, -1, 0);
        if (got != want) {
            // Another checker library of this process (each has its own copy of this stand-in) may
            // have left the range mapped, e.g. after a test that failed half way: its contents are
            // stale by then, so the range is taken over.
            if (got != MAP_FAILED) munmap(got, grow_to - s.mapped_end);
            got = mmap(want, grow_to - s.mapped_end, PROT_READ | PROT_WRITE,
                       MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
        }
        if (got != want) {
            fprintf(stderr, "torpor_ref_fake: cannot map canonical device range at %p\n", want);
            abort();
        }
        s.mapped_end = grow_to;
    }
    s.bump = off + need;
    return (void*)(base + off);
}

// Drop every fake device mapping and restart the bump allocators.
inline void reset_world() {
    World& w = world();
    std::lock_guard<std::mutex> g(w.mu);
    for (int d = 0; d < kMaxDev; ++d) {
        if (w.dev[d].mapped_end) {
            munmap((void*)(kCanonBase + (uint64_t)d * kCanonStride), w.dev[d].mapped_end);
        }
        w.dev[d] = DevSpace();
    }
}

}  // namespace torpor_ref_fake

inline const char* cudaGetErrorString(cudaError_t e) { return e == 0 ? "no error" : "fake cuda error"; }
inline cudaError_t cudaSetDevice(int d) { torpor_ref_fake::cur_device() = d; return cudaSuccess; }
inline cudaError_t cudaGetDevice(int* d) { *d = torpor_ref_fake::cur_device(); return cudaSuccess; }
inline cudaError_t cudaMalloc(void** p, size_t size) {
    *p = torpor_ref_fake::dev_alloc(size);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
template <class T> inline cudaError_t cudaMalloc(T** p, size_t size) { return cudaMalloc((void**)p, size); }
inline cudaError_t cudaFree(void*) { return cudaSuccess; }  // address space is never reused
inline cudaError_t cudaMallocHost(void** p, size_t size) {
    *p = aligned_alloc(4096, (size + 4095) / 4096 * 4096);
    return *p ? cudaSuccess : cudaErrorMemoryAllocation;
}
inline cudaError_t cudaFreeHost(void* p) { free(p); return cudaSuccess; }
inline cudaError_t cudaMemcpy(void* dst, const void* src, size_t n, cudaMemcpyKind) { memcpy(dst, src, n); return cudaSuccess; }
inline cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t n, cudaMemcpyKind, cudaStream_t = nullptr) { memcpy(dst, src, n); return cudaSuccess; }
inline cudaError_t cudaMemcpyPeerAsync(void* dst, int, const void* src, int, size_t n, cudaStream_t = nullptr) { memcpy(dst, src, n); return cudaSuccess; }
inline cudaError_t cudaMemsetAsync(void* p, int v, size_t n, cudaStream_t = nullptr) { memset(p, v, n); return cudaSuccess; }
inline cudaError_t cudaStreamCreateWithPriority(cudaStream_t* s, unsigned int, int) { *s = nullptr; return cudaSuccess; }
inline cudaError_t cudaEventCreate(cudaEvent_t* e) { *e = nullptr; return cudaSuccess; }
inline cudaError_t cudaEventRecord(cudaEvent_t, cudaStream_t = nullptr) { return cudaSuccess; }
inline cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
inline cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
inline cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }

#endif  // TORPOR_REF_FAKE_CUDA

#ifdef TORPOR_REF_WITH_CONTROLLER
// What include/server/controller.hpp needs beyond the swap-path headers: the signal messages
// (proto/signal.proto, normally protoc-generated), a cuDNN handle and two peer-access calls.
namespace signal {
enum RequestType { ExecuteAfterLoad = 0, Execute = 1, Load = 2, Unload = 3, ExecuteForRecord = 10, Replay = 11 };
enum AckType { OK = 0, Inavail = 1 };
inline int format_as(RequestType t) { return (int)t; }   // how the logger prints it
inline int format_as(AckType t) { return (int)t; }
struct SignalRequest {
    RequestType type_ = ExecuteAfterLoad;
    std::string function_, payload_;
    // the harness's own encoding of a scripted request: "<type> <function> <payload>"
    bool ParseFromString(const std::string& s) {
        size_t a = s.find(' '), b = s.find(' ', a + 1);
        type_ = (RequestType)atoi(s.substr(0, a).c_str());
        function_ = s.substr(a + 1, b - a - 1);
        payload_ = s.substr(b + 1);
        return true;
    }
    RequestType type() const { return type_; }
    const std::string& function() const { return function_; }
    const std::string& payload() const { return payload_; }
};
struct SignalAck {
    int ack_ = 0, resp_ = 0;
    void set_ack(AckType a) { ack_ = (int)a; }
    void set_resp(int r) { resp_ = r; }
    bool SerializeToString(std::string* out) const {
        *out = std::to_string(ack_) + " " + std::to_string(resp_);
        return true;
    }
};
}  // namespace signal
using signal::RequestType;
using signal::SignalRequest;
using signal::AckType;
using signal::SignalAck;

typedef void* cudnnHandle_t;
typedef int cudnnStatus_t;
static const cudnnStatus_t CUDNN_STATUS_SUCCESS = 0;
inline cudnnStatus_t cudnnCreate(cudnnHandle_t* h) { *h = nullptr; return CUDNN_STATUS_SUCCESS; }
#define cudnnCheck(ans) { (void)(ans); }
#ifdef TORPOR_REF_FAKE_CUDA
namespace torpor_ref_fake { inline int& device_count() { static int n = 4; return n; } }
inline cudaError_t cudaGetDeviceCount(int* n) { *n = torpor_ref_fake::device_count(); return cudaSuccess; }
inline cudaError_t cudaDeviceCanAccessPeer(int* can, int, int) { *can = 0; return cudaSuccess; }
inline cudaError_t cudaDeviceEnablePeerAccess(int, unsigned int) { return cudaSuccess; }
#endif
#endif  // TORPOR_REF_WITH_CONTROLLER

#ifdef TORPOR_REF_WITH_EXECUTOR
// What include/server/cuda_server.hpp (the executor) needs beyond the swap-path headers: the
// message classes (stand-ins generated from the reference's .proto files by gen_pb_shim.py),
// cuDNN / cuBLAS names, and the rest of the CUDA calls its services make.  Only the memory
// services and the kernel launch are exercised; everything else merely has to compile.
#ifndef TORPOR_REF_FAKE_CUDA
// the executor against the real runtime (tests/executor_gpu_probe.cpp): its driver-API services need
// <cuda.h>, and its logger prints a cudaMemcpyKind
#include <cuda.h>
inline int format_as(cudaMemcpyKind k) { return (int)k; }
#endif
#include "cudarpc.pb.h"
#include "signal.pb.h"
#include "cudarpc.using.h"
#include "signal.using.h"
#include <set>

typedef void* cudnnHandle_t;
typedef void* cudnnTensorDescriptor_t;
typedef void* cudnnFilterDescriptor_t;
typedef void* cudnnConvolutionDescriptor_t;
typedef int cudnnStatus_t;
typedef int cudnnDataType_t;
typedef int cudnnTensorFormat_t;
typedef int cudnnMathType_t;
typedef int cudnnConvolutionMode_t;
typedef int cudnnConvolutionFwdAlgo_t;
typedef int cudnnBatchNormMode_t;
struct cudnnConvolutionFwdAlgoPerf_t { int algo = 0; int status = 0; float time = 0; size_t memory = 0; int determinism = 0; int mathType = 0; int reserved[3] = {0, 0, 0}; };
static const cudnnStatus_t CUDNN_STATUS_SUCCESS = 0;
typedef void* cublasHandle_t;
typedef int cublasStatus_t;
typedef int cublasOperation_t;
typedef int cublasMath_t;
#define TORPOR_STUB(name) inline int name(...) { return 0; }   /* C variadic: some calls pass variable-length arrays */
TORPOR_STUB(cudnnCreate) TORPOR_STUB(cudnnDestroy) TORPOR_STUB(cudnnSetStream)
TORPOR_STUB(cudnnCreateTensorDescriptor) TORPOR_STUB(cudnnSetTensorNdDescriptor) TORPOR_STUB(cudnnDestroyTensorDescriptor)
TORPOR_STUB(cudnnCreateFilterDescriptor) TORPOR_STUB(cudnnSetFilterNdDescriptor) TORPOR_STUB(cudnnDestroyFilterDescriptor)
TORPOR_STUB(cudnnCreateConvolutionDescriptor) TORPOR_STUB(cudnnSetConvolutionNdDescriptor) TORPOR_STUB(cudnnDestroyConvolutionDescriptor)
TORPOR_STUB(cudnnSetConvolutionGroupCount) TORPOR_STUB(cudnnSetConvolutionMathType) TORPOR_STUB(cudnnGetConvolutionForwardAlgorithm_v7)
TORPOR_STUB(cudnnConvolutionForward) TORPOR_STUB(cudnnBatchNormalizationForwardInference)
TORPOR_STUB(cublasCreate) TORPOR_STUB(cublasDestroy) TORPOR_STUB(cublasSetStream) TORPOR_STUB(cublasSetMathMode)
TORPOR_STUB(cublasGetMathMode) TORPOR_STUB(cublasSgemm) TORPOR_STUB(cublasSgemmStridedBatched)
#define cudnnCheck(ans) { (void)(ans); }

#ifdef TORPOR_REF_FAKE_CUDA
typedef int CUresult;
typedef int CUdevice;
typedef int cudaDeviceAttr;
typedef int cudaStreamCaptureStatus;
static const unsigned int cudaStreamDefault = 0;
struct cudaDeviceProp { char name[256]; size_t totalGlobalMem; int major, minor, multiProcessorCount; };
struct dim3 { unsigned int x, y, z; dim3(unsigned int a = 1, unsigned int b = 1, unsigned int c = 1) : x(a), y(b), z(c) {} };
TORPOR_STUB(cuInit) TORPOR_STUB(cuDriverGetVersion) TORPOR_STUB(cuDevicePrimaryCtxGetState)
TORPOR_STUB(cudaDriverGetVersion) TORPOR_STUB(cudaRuntimeGetVersion) TORPOR_STUB(cudaGetLastError)
TORPOR_STUB(cudaDeviceGetAttribute) TORPOR_STUB(cudaStreamCreate) TORPOR_STUB(cudaStreamCreateWithFlags)
TORPOR_STUB(cudaStreamIsCapturing) TORPOR_STUB(cudaStreamGetCaptureInfo) TORPOR_STUB(cudaGetSymbolAddress)
TORPOR_STUB(cudaEventCreateWithFlags) TORPOR_STUB(cudaEventQuery)
inline cudaError_t cudaGetDeviceProperties(cudaDeviceProp* p, int) { memset(p, 0, sizeof(*p)); return cudaSuccess; }
namespace torpor_ref_fake { inline int& device_count() { static int n = 4; return n; } }
inline cudaError_t cudaGetDeviceCount(int* n) { *n = torpor_ref_fake::device_count(); return cudaSuccess; }
inline cudaError_t cudaDeviceCanAccessPeer(int* can, int, int) { *can = 0; return cudaSuccess; }
inline cudaError_t cudaDeviceEnablePeerAccess(int, unsigned int) { return cudaSuccess; }
// A launch is not run: the harness keeps the kernel and the argument words the executor passed.
namespace torpor_ref_fake { void record_launch(const void* func, void** args); }
inline cudaError_t cudaLaunchKernel(const void* func, dim3, dim3, void** args, size_t, cudaStream_t) {
    torpor_ref_fake::record_launch(func, args);
    return cudaSuccess;
}
#endif
#endif  // TORPOR_REF_WITH_EXECUTOR

#define cudaCheck(ans) { cudaAssert((ans), __FILE__, __LINE__); }
inline void cudaAssert(cudaError_t err, const char* file, int line, bool abort_flag = false) {
    if (err != cudaSuccess) {
        fprintf(stderr, "cuda assert: %s %s %d\n", cudaGetErrorString(err), file, line);
        if (abort_flag) assert(0);
    }
}

#endif  // TORPOR_REF_SHIM_CUDA_COMMON_HPP_
