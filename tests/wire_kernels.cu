// TEST SUPPORT: two small kernels and a launch-by-name entry, standing in for the generated
// kernel table of the reference's executor (lookup(), src/server/kernel_lookup.cpp).  The wire
// tests give WireExecutor these launchers, so that a serialised cudaLaunchKernelQuery ends in a
// real cudaLaunchKernel on the argument words the executor rewrote.
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>

extern "C" __global__ void wire_saxpy(const float* w, const float* x, float* y, uint64_t n, float a) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        y[i] = a * w[i] + x[i];
}

// One argument that is a struct of two pointers and a count: the executor rewrites pointer words
// inside an argument, not only whole arguments (cuda_server.hpp:1250-1257).
struct WirePair {
    const float* w;
    float* y;
    uint64_t n;
};
extern "C" __global__ void wire_scale_pair(WirePair p, float a) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < p.n; i += (uint64_t)gridDim.x * blockDim.x)
        p.y[i] = a * p.w[i];
}

// cudaLaunchKernel of the kernel called `name` on the legacy default stream of the current
// device.  args[i] points at the bytes of argument i.  Returns the CUDA error code, -1 for an
// unknown name.
extern "C" int wire_launch(const char* name, void** args, unsigned grid, unsigned block, unsigned long long shared_mem) {
    const void* fn = nullptr;
    if (!strcmp(name, "wire_saxpy")) fn = (const void*)wire_saxpy;
    else if (!strcmp(name, "wire_scale_pair")) fn = (const void*)wire_scale_pair;
    if (!fn) return -1;
    return (int)cudaLaunchKernel(fn, dim3(grid), dim3(block), args, (size_t)shared_mem, (cudaStream_t)0);
}
