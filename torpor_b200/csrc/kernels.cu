// sm_100a kernels of the swap engine.
//
// place_kernel is the one data mover: a persistent grid walks the tiles of a
// swap in first-run access order, copies each tile with 16-byte vector
// loads/stores, and -- fused into the same kernel -- counts finished tiles per
// parameter; whoever finishes a parameter's last tile rewrites its row of the
// device-pointer table (rebound address, readiness) and the host-visible mirror
// of that row.  It replaces, in the reference, the per-parameter
// cudaMemcpyAsync / cudaMemcpyPeerAsync loop with its host-side staging copy and
// per-group event round trip (include/server/memory_manager.hpp:311-329,
// 375-409,441-449).  Source and destination may each be page-locked host memory
// (read or written across PCIe by the SMs), this GPU's pool, or a peer GPU's pool
// across NVLink; nothing in it waits on another kernel.
//
// The work is byte movement bound by PCIe, NVLink or HBM; there is no
// contraction in it, so no tensor-core path.

#include "kernels.hpp"

#include <cstring>
#include <mutex>
#include <string>

#include "../../include/torpor_swap.h"

namespace tsw {
int fail(int code, const std::string& msg);  // records the thread's last error text (engine.cpp)
}

namespace tsw {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 8;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
#ifndef TSW_LD16
#define TSW_LD16 "ld.global.nc.L1::no_allocate.v4.u32"
#endif
    asm(TSW_LD16 " {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Bytes [0, len) from src to dst where src and dst are congruent modulo 16.
__device__ __forceinline__ void copy_span16(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                            uint32_t len) {
    const uint32_t tid = threadIdx.x;
    uint32_t head = (16u - (uint32_t)((uintptr_t)dst & 15u)) & 15u;
    if (head > len) head = len;
    if (tid < head) dst[tid] = src[tid];
    const uint32_t n16 = (len - head) >> 4;
    const uint8_t* s = src + head;
    uint8_t* d = dst + head;
    for (uint32_t i = tid; i < n16; i += kThreads * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint32_t idx = i + u * kThreads;
            if (idx < n16) v[u] = ld_stream16(s + ((size_t)idx << 4));
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            uint32_t idx = i + u * kThreads;
            if (idx < n16) st_stream16(d + ((size_t)idx << 4), v[u]);
        }
    }
    const uint32_t done = head + (n16 << 4);
    const uint32_t tail = len - done;
    if (tid < tail) dst[done + tid] = src[done + tid];
}

// Same for the rare case of a source and destination that disagree modulo 16:
// fall back to the widest word both sides can be aligned to.
template <typename T>
__device__ __forceinline__ void copy_span_narrow(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                 uint32_t len) {
    constexpr uint32_t W = sizeof(T);
    const uint32_t tid = threadIdx.x;
    uint32_t head = (W - (uint32_t)((uintptr_t)dst & (W - 1))) & (W - 1);
    if (head > len) head = len;
    if (tid < head) dst[tid] = src[tid];
    const uint32_t n = (len - head) / W;
    const T* s = reinterpret_cast<const T*>(src + head);
    T* d = reinterpret_cast<T*>(dst + head);
    for (uint32_t i = tid; i < n; i += kThreads) d[i] = s[i];
    const uint32_t done = head + n * W;
    const uint32_t tail = len - done;
    if (tid < tail) dst[done + tid] = src[done + tid];
}

__device__ __forceinline__ void copy_span(uint64_t src, uint64_t dst, uint32_t len) {
    const uint8_t* s = reinterpret_cast<const uint8_t*>(src);
    uint8_t* d = reinterpret_cast<uint8_t*>(dst);
    const uint32_t diff = (uint32_t)((src ^ dst) & 15u);
    if (diff == 0) copy_span16(s, d, len);
    else if ((diff & 7u) == 0) copy_span_narrow<uint2>(s, d, len);
    else if ((diff & 3u) == 0) copy_span_narrow<uint32_t>(s, d, len);
    else if ((diff & 1u) == 0) copy_span_narrow<uint16_t>(s, d, len);
    else copy_span_narrow<uint8_t>(s, d, len);
}

// Largest k in [0, n) with first[k] <= t (first[] is non-decreasing, first[0] == 0).
__device__ __forceinline__ uint32_t owner_of_tile(const uint32_t* first, uint32_t n, uint32_t t) {
    uint32_t lo = 0, hi = n;
    while (hi - lo > 1) {
        uint32_t mid = (lo + hi) >> 1;
        if (first[mid] <= t) lo = mid;
        else hi = mid;
    }
    return lo;
}

// Copy tile t and, when asked to, count it towards its row; the CTA that completes a row
// rewrites that row of the pointer table.  Every thread of the CTA calls this with the same t.
__device__ __forceinline__ void move_tile(const PlaceArgs& a, const uint32_t* s_first, uint32_t t) {
    const uint32_t k = owner_of_tile(s_first, a.n_descs, t);
    const PlaceDesc d = a.descs[k];
    const uint64_t off = (uint64_t)(t - s_first[k]) * a.tile_bytes;
    if (off >= d.bytes) {  // table and tile numbering disagree: report, move nothing
        if (threadIdx.x == 0 && a.status) *reinterpret_cast<volatile uint32_t*>(a.status) = 1u;
        return;
    }
    if (a.skip_min_bytes && d.bytes >= a.skip_min_bytes) return;   // the copy engine's share
    const uint64_t left = d.bytes - off;
    const uint32_t len = left < a.tile_bytes ? (uint32_t)left : a.tile_bytes;
    copy_span(d.src + off, d.dst + off, len);

    if (a.done_count) {
        if (a.system_scope) __threadfence_system();
        else __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t before = a.system_scope ? atomicAdd_system(&a.done_count[d.row], 1u)
                                                   : atomicAdd(&a.done_count[d.row], 1u);
            if (before + 1 == d.row_tiles) {
                // Last tile of this parameter -- the others may have been moved by other
                // segments, launches or GPUs: re-arm the counter, rebind the table row,
                // then raise the flag.  ONE system-scope fence, between the address and the
                // flag: a reader that sees the flag must see the address (the bytes were
                // fenced before the count above).  The re-armed counter is next read by a
                // later swap's kernels, which the host launches only after this kernel has
                // drained; nothing follows the flag.  A fence after a store to host-mapped
                // memory costs a trip across a PCIe link whose read queue this very kernel
                // keeps full, and the CTA waits for this thread at its next tile: with three
                // fences per row a 32-CTA swap of 391 rows spent 0.7 ms of 13.9 ms in them.
                a.done_count[d.row] = 0;
                a.table_phys[d.row] = d.row_dst;
                if (a.host_phys) a.host_phys[d.row] = d.row_dst;
                __threadfence_system();
                a.table_flag[d.row] = a.flag_value;
                if (a.host_flag) a.host_flag[d.row] = a.host_flag_value;
                if (a.host_gen) a.host_gen[d.row] = a.flag_value;
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads) place_kernel(const PlaceArgs a) {
    extern __shared__ uint32_t s_first[];  // n_descs + 1 tile prefix sums
    for (uint32_t i = threadIdx.x; i <= a.n_descs; i += kThreads) s_first[i] = a.first_tile[i];
    __syncthreads();

    if (a.ticket == nullptr) {
        const uint64_t step = (uint64_t)gridDim.x * a.tile_stride;
        for (uint64_t t64 = a.tile_lo + (uint64_t)blockIdx.x * a.tile_stride; t64 < a.tile_hi; t64 += step)
            move_tile(a, s_first, (uint32_t)t64);
        return;
    }
    // Dynamic dealing.  The counter starts at tile_lo and only grows; a CTA that draws a
    // number at or beyond tile_hi is done, so the loop ends after at most one failed draw.
    __shared__ uint32_t s_draw;
    for (;;) {
        if (threadIdx.x == 0) s_draw = atomicAdd_system(a.ticket, a.ticket_chunk);
        __syncthreads();
        const uint32_t first = s_draw;
        __syncthreads();
        if (first >= a.tile_hi) break;
        const uint32_t last = (a.tile_hi - first < a.ticket_chunk) ? a.tile_hi : first + a.ticket_chunk;
        for (uint32_t t = first; t < last; ++t) move_tile(a, s_first, t);
    }
}

// The publish step alone.  One thread per segment of [lo, hi); the bytes were moved by a copy
// that precedes this kernel in its stream, so they are complete when it runs.
__global__ void publish_rows_kernel(const PlaceArgs a, uint32_t lo, uint32_t hi) {
    const uint32_t k = lo + blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= hi) return;
    const PlaceDesc d = a.descs[k];
    a.table_phys[d.row] = d.row_dst;
    if (a.host_phys) a.host_phys[d.row] = d.row_dst;
    __threadfence_system();
    a.table_flag[d.row] = a.flag_value;
    if (a.host_flag) a.host_flag[d.row] = a.host_flag_value;
    if (a.host_gen) a.host_gen[d.row] = a.flag_value;
    __threadfence_system();
}

// ------------------------------------------------------------------ bulk-copy mover
//
// The same placement, moved by the bulk asynchronous copy unit instead of by loads and
// stores of the SMs' threads: one thread per CTA keeps a ring of shared-memory stages; each
// 16 KiB chunk of a tile is fetched with cp.async.bulk (global -> shared, completion counted
// on an mbarrier) and written out with cp.async.bulk (shared -> global, bulk group).  No
// multicast, no cluster: every CTA fetches its own chunks.  Needs source, destination and
// chunk sizes to be multiples of 16 bytes; a ragged tail of a tile (< 16 B) is copied by
// the thread itself.  Every wait is bounded: when an mbarrier does not complete within
// kSpinLimit polls the CTA records status 2, drains what it has in flight and stops.
constexpr int kBulkThreads = 32;
constexpr uint32_t kBulkChunk = 16u * 1024;
constexpr int kBulkStages = 4;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the barrier did not flip within the limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, uint64_t gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(uint64_t gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async;" ::: "memory"); }

__global__ void __launch_bounds__(kBulkThreads) place_kernel_bulk(const PlaceArgs a) {
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    unsigned char* stage = bulk_smem;
    uint64_t* bar = reinterpret_cast<uint64_t*>(bulk_smem + kBulkStages * kBulkChunk);
    uint32_t* s_first = reinterpret_cast<uint32_t*>(bulk_smem + kBulkStages * kBulkChunk + 64);
    for (uint32_t i = threadIdx.x; i <= a.n_descs; i += kBulkThreads) s_first[i] = a.first_tile[i];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkStages; ++s) mbar_init(&bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    __syncwarp();
    if (threadIdx.x != 0) return;   // one thread drives the copy unit; the warp only loaded the table

    uint32_t parity = 0;            // bit s = phase the next wait on stage s expects
    bool failed = false;
    const uint64_t step = (uint64_t)gridDim.x * a.tile_stride;
    uint64_t next = a.tile_lo + (uint64_t)blockIdx.x * a.tile_stride;
    uint32_t drawn = 0, drawn_end = 0;
    for (;;) {
        uint32_t t;
        if (a.ticket) {
            if (drawn == drawn_end) {
                drawn = atomicAdd_system(a.ticket, a.ticket_chunk);
                if (drawn >= a.tile_hi) break;
                drawn_end = (a.tile_hi - drawn < a.ticket_chunk) ? a.tile_hi : drawn + a.ticket_chunk;
            }
            t = drawn++;
        } else {
            if (next >= a.tile_hi) break;
            t = (uint32_t)next;
            next += step;
        }
        const uint32_t k = owner_of_tile(s_first, a.n_descs, t);
        const PlaceDesc d = a.descs[k];
        const uint64_t off = (uint64_t)(t - s_first[k]) * a.tile_bytes;
        if (off >= d.bytes) {
            if (a.status) *reinterpret_cast<volatile uint32_t*>(a.status) = 1u;
            continue;
        }
        if (a.skip_min_bytes && d.bytes >= a.skip_min_bytes) continue;   // the copy engine's share
        const uint64_t left = d.bytes - off;
        const uint32_t len = left < a.tile_bytes ? (uint32_t)left : a.tile_bytes;
        const uint32_t body = len & ~15u;
        const uint32_t n_chunks = (body + kBulkChunk - 1) / kBulkChunk;
        const uint64_t src = d.src + off, dst = d.dst + off;

        const uint32_t ahead = n_chunks < (uint32_t)kBulkStages ? n_chunks : (uint32_t)kBulkStages;
        for (uint32_t c = 0; c < ahead; ++c) {
            const uint32_t bytes = (body - c * kBulkChunk) < kBulkChunk ? (body - c * kBulkChunk) : kBulkChunk;
            mbar_expect_tx(&bar[c], bytes);
            bulk_load(stage + c * kBulkChunk, src + (uint64_t)c * kBulkChunk, bytes, &bar[c]);
        }
        uint32_t in_flight_lo = 0, in_flight_hi = ahead;   // loads issued and not yet waited for: [lo, hi)
        for (uint32_t c = 0; c < n_chunks; ++c) {
            const uint32_t s = c % kBulkStages;
            const uint32_t bytes = (body - c * kBulkChunk) < kBulkChunk ? (body - c * kBulkChunk) : kBulkChunk;
            if (!mbar_wait_bounded(&bar[s], (parity >> s) & 1u)) {
                failed = true;
                break;
            }
            parity ^= 1u << s;
            in_flight_lo = c + 1;
            fence_async_proxy();
            bulk_store(dst + (uint64_t)c * kBulkChunk, stage + s * kBulkChunk, bytes);
            bulk_commit();
            const uint32_t n = c + kBulkStages;
            if (n < n_chunks) {
                bulk_wait_read_all();   // the stage is free again once the store has read it
                const uint32_t nb = (body - n * kBulkChunk) < kBulkChunk ? (body - n * kBulkChunk) : kBulkChunk;
                mbar_expect_tx(&bar[s], nb);
                bulk_load(stage + s * kBulkChunk, src + (uint64_t)n * kBulkChunk, nb, &bar[s]);
                in_flight_hi = n + 1;
            }
        }
        if (failed) {
            // give the loads still in flight one more bounded chance to land, then stop
            for (uint32_t c = in_flight_lo; c < in_flight_hi; ++c) {
                const uint32_t s = c % kBulkStages;
                if (mbar_wait_bounded(&bar[s], (parity >> s) & 1u)) parity ^= 1u << s;
            }
            bulk_wait_all();
            if (a.status) *reinterpret_cast<volatile uint32_t*>(a.status) = 2u;
            return;
        }
        for (uint32_t i = body; i < len; ++i)   // ragged tail, fewer than 16 bytes
            reinterpret_cast<uint8_t*>(dst)[i] = reinterpret_cast<const uint8_t*>(src)[i];
        bulk_wait_all();
        fence_async_proxy();

        if (a.done_count) {
            __threadfence_system();
            const uint32_t before = atomicAdd_system(&a.done_count[d.row], 1u);
            if (before + 1 == d.row_tiles) {
                a.done_count[d.row] = 0;
                __threadfence_system();
                a.table_phys[d.row] = d.row_dst;
                if (a.host_phys) a.host_phys[d.row] = d.row_dst;
                __threadfence_system();
                a.table_flag[d.row] = a.flag_value;
                if (a.host_flag) a.host_flag[d.row] = a.host_flag_value;
                if (a.host_gen) a.host_gen[d.row] = a.flag_value;
                __threadfence_system();
            }
        }
    }
}

// ------------------------------------------------------------------ checksum

__device__ __forceinline__ uint32_t load_word(const uint8_t* base, uint64_t byte_off, uint64_t total, bool aligned) {
    if (aligned && byte_off + 4 <= total) return *reinterpret_cast<const uint32_t*>(base + byte_off);
    uint32_t w = 0;
    for (int b = 0; b < 4; ++b)
        if (byte_off + b < total) w |= (uint32_t)base[byte_off + b] << (8 * b);
    return w;
}

__global__ void __launch_bounds__(kThreads) checksum_kernel(const SumDesc* descs, uint32_t n_descs,
                                                            uint32_t total_tiles, uint32_t tile_bytes,
                                                            unsigned long long* out) {
    __shared__ unsigned long long red[2][kThreads / 32];
    for (uint32_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
        uint32_t lo = 0, hi = n_descs;
        while (hi - lo > 1) {
            uint32_t mid = (lo + hi) >> 1;
            if (descs[mid].first_tile <= t) lo = mid;
            else hi = mid;
        }
        const SumDesc d = descs[lo];
        const uint64_t off = (uint64_t)(t - d.first_tile) * tile_bytes;
        unsigned long long s1 = 0, s2 = 0;
        if (off < d.bytes) {
            const uint64_t left = d.bytes - off;
            const uint64_t len = left < tile_bytes ? left : tile_bytes;
            const uint64_t n_words = (len + 3) >> 2;
            const uint8_t* base = reinterpret_cast<const uint8_t*>(d.addr);
            const bool aligned = (d.addr & 3ull) == 0;
            const uint64_t word0 = off >> 2;
            for (uint64_t i = threadIdx.x; i < n_words; i += kThreads) {
                const unsigned long long w = load_word(base, off + (i << 2), d.bytes, aligned);
                s1 += w;
                s2 += (word0 + i + 1ull) * w;
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            s1 += __shfl_down_sync(0xffffffffu, s1, o);
            s2 += __shfl_down_sync(0xffffffffu, s2, o);
        }
        if ((threadIdx.x & 31) == 0) {
            red[0][threadIdx.x >> 5] = s1;
            red[1][threadIdx.x >> 5] = s2;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long a1 = 0, a2 = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                a1 += red[0][w];
                a2 += red[1][w];
            }
            atomicAdd(&out[2 * d.row], a1);
            atomicAdd(&out[2 * d.row + 1], a2);
        }
        __syncthreads();
    }
}

}  // namespace

int default_grid_ctas(int device) {
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    // 58 registers x 256 threads keep 4 CTAs resident per SM; six per SM in the grid (two queued
    // behind the resident four) measured best for HBM-to-HBM moves: fewer concurrent streams keep
    // DRAM rows open, the queued CTAs fill the tail.  Forcing 5 or 6 resident CTAs per SM with a
    // register bound was 8-25 % slower.  PCIe-bound moves do not depend on the grid.
    return sms * 6;
}

int default_grid_ctas_host(int device) {
    // A move across PCIe is bound by the link whatever the grid: measured, 8 CTAs already read the
    // host store at the link's full rate, and 12 to 888 differ by about 1 %.  But every resident CTA
    // holds a quarter of its SM's registers until the swap is over, and a large matrix-product
    // kernel wants a whole SM: with 148 CTAs or more the swapped-in function's first kernels did
    // not start before the swap had finished (a loop of products beside the swap took 1.95 x as
    // long); with 32 CTAs it took 1.43 x, with 16 CTAs 1.21 x.  On the 13.5 GB Llama-shaped set 32
    // CTAs are level with 888 (262.3 against 262.4 ms); sets of many small tensors land 2-3 % later
    // (BERT-large 13.34 against 13.07 ms).  A small grid also keeps the tiles in flight within 2 MiB
    // of the access order, so parameters arrive in the order the first inference needs them
    // instead of all at the end.
    (void)device;
    return 32;
}

cudaError_t launch_place(const PlaceArgs& a, int grid_ctas, cudaStream_t stream, int mover) {
    if (a.n_descs == 0 || a.tile_hi <= a.tile_lo) return cudaSuccess;
    if (a.tile_bytes == 0 || (a.tile_bytes & 15u) || a.tile_stride == 0) return cudaErrorInvalidValue;
    if (a.ticket && a.ticket_chunk == 0) return cudaErrorInvalidValue;
    if (mover == 1) {
        const uint64_t tiles = a.ticket ? (uint64_t)(a.tile_hi - a.tile_lo)
                                        : ((uint64_t)(a.tile_hi - a.tile_lo) + a.tile_stride - 1) / a.tile_stride;
        int g = grid_ctas > 0 ? grid_ctas : 444;
        if ((uint64_t)g > tiles) g = (int)tiles;
        const size_t bytes = (size_t)kBulkStages * kBulkChunk + 64 + sizeof(uint32_t) * ((size_t)a.n_descs + 1);
        if (bytes > 200 * 1024) return cudaErrorInvalidValue;
        cudaError_t e = cudaFuncSetAttribute(place_kernel_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        place_kernel_bulk<<<g, kBulkThreads, bytes, stream>>>(a);
        return cudaGetLastError();
    }
    const uint64_t mine = a.ticket ? (uint64_t)(a.tile_hi - a.tile_lo)
                                   : ((uint64_t)(a.tile_hi - a.tile_lo) + a.tile_stride - 1) / a.tile_stride;
    int grid = grid_ctas > 0 ? grid_ctas : 888;
    if ((uint64_t)grid > mine) grid = (int)mine;
    const size_t smem = sizeof(uint32_t) * ((size_t)a.n_descs + 1);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    place_kernel<<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_publish_rows(const PlaceArgs& a, uint32_t lo, uint32_t hi, cudaStream_t stream) {
    if (hi <= lo) return cudaSuccess;
    if (!a.table_phys || !a.table_flag) return cudaErrorInvalidValue;
    const uint32_t n = hi - lo;
    publish_rows_kernel<<<(n + 63) / 64, 64, 0, stream>>>(a, lo, hi);
    return cudaGetLastError();
}

cudaError_t launch_checksum(const SumDesc* descs, uint32_t n_descs, uint32_t total_tiles, uint32_t tile_bytes,
                            unsigned long long* out, int grid_ctas, cudaStream_t stream) {
    if (n_descs == 0 || total_tiles == 0) return cudaSuccess;
    int grid = grid_ctas > 0 ? grid_ctas : 592;
    if ((uint32_t)grid > total_tiles) grid = (int)total_tiles;
    checksum_kernel<<<grid, kThreads, 0, stream>>>(descs, n_descs, total_tiles, tile_bytes, out);
    return cudaGetLastError();
}

}  // namespace tsw

// =====================================================================================
// tsw_place_segments_static: the placement mover for callers that must not allocate.
//
// Who that is: code running inside a GPU-sharing server once it is in steady state.  A
// remoting executor that forwards a client's intercepted CUDA calls, a plugin loaded
// into a process whose device memory has been handed over to the block pool in full, or
// a helper rank that only lends its PCIe link to a sharded swap, cannot afford a device
// allocation on the swap path: cudaMalloc synchronises the whole device (stalling the
// inference kernels that share it), may fail because the pool already owns the memory,
// and in an interposed process may be routed back to the very server that is calling.
// tsw_place_segments grows a device-side descriptor table with cudaMalloc and a pinned
// staging buffer with cudaHostAlloc; this variant keeps the same table in a fixed
// array that is part of the loaded module instead.
//
// The scratch: kStaticScratchBytes (1 MiB) of device memory per GPU that loads this
// library, held until the process exits.  It bounds one call to kStaticMaxSegments
// segments.  Every call on a device uses the same array and finds the previous call's
// table in it; a call rewrites all of the table it uses, so nothing needs clearing, but
// two calls whose work overlaps on the GPU (different streams, or several host threads)
// overwrite each other's table: keep calls on one device in one stream, or serialise them.
//
// The array's name below is only meaningful in device code.  Host code must not pass it
// to a kernel: the host-side symbol is a stand-in, not a device address.  The address is
// looked up once per device, with that device current, by cudaGetSymbolAddress; that
// happens in the first call made for a device, so make that first call outside of any
// stream capture.  The address is cached for the life of the process: it does not survive
// a cudaDeviceReset of that device.  Every call uploads its table from host arrays that
// belong to the library and are reused by the next call on that device.  Calls lock per
// device, and the caller's current device is the same after the call as before it.
namespace tsw {
namespace {

constexpr uint32_t kStaticMaxSegments = 16384;
constexpr size_t kStaticDescBytes = sizeof(PlaceDesc) * kStaticMaxSegments;              // 640 KiB
constexpr size_t kStaticFirstBytes = sizeof(uint32_t) * (kStaticMaxSegments + 1);        // 64 KiB + 4
constexpr size_t kStaticScratchBytes = 1u << 20;
static_assert(kStaticDescBytes + kStaticFirstBytes <= kStaticScratchBytes, "static scratch too small");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
// Where the kernel reports a table that does not fit its tile numbering (the sign of two calls
// that overlapped on the GPU and overwrote each other's table); read by tsw_place_segments_static_status.
static __device__ __align__(256) uint32_t g_static_status[64];

constexpr int kMaxDevices = 16;

// Per device: the device addresses of the two arrays above, a lock, and the host-side staging
// of one call's table -- so a caller blocked on one GPU's stream does not hold up callers on others.
struct StaticDevice {
    std::mutex mu;
    bool known = false;
    unsigned char* scratch = nullptr;
    uint32_t* status = nullptr;
    PlaceDesc host_descs[kStaticMaxSegments];
    uint32_t host_first[kStaticMaxSegments + 1];
};
StaticDevice g_static_dev[kMaxDevices];

// Puts the caller's current device back when the entry point returns.
struct DeviceRestore {
    int prev = -1;
    DeviceRestore() { if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; cudaGetLastError(); } }
    ~DeviceRestore() { if (prev >= 0) cudaSetDevice(prev); }
};

// Set-up, once per device, with that device current: the device addresses of the arrays.
int static_setup(StaticDevice& sd) {
    if (sd.known) return TSW_OK;
    unsigned char* p = nullptr;
    uint32_t* st = nullptr;
    cudaError_t err = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (err != cudaSuccess || !p)
        return fail(TSW_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(err));
    err = cudaGetSymbolAddress((void**)&st, g_static_status);
    if (err != cudaSuccess || !st)
        return fail(TSW_ERR_CUDA, std::string("cudaGetSymbolAddress(static status): ") + cudaGetErrorString(err));
    sd.scratch = p;
    sd.status = st;
    sd.known = true;
    return TSW_OK;
}

}  // namespace
}  // namespace tsw

extern "C" int tsw_place_segments_static(int device, const tsw_segment* segs, int n, uint32_t tile_bytes,
                                         uint32_t tile_first, uint32_t tile_stride, const tsw_publish* pub,
                                         void* stream) {
    using namespace tsw;
    static_assert(sizeof(tsw_segment) == sizeof(PlaceDesc), "segment layout");
    if (n < 0 || (n > 0 && !segs)) return fail(TSW_ERR_INVALID, "bad segment list");
    if (device < 0 || device >= kMaxDevices) return fail(TSW_ERR_INVALID, "device ordinal out of range");
    if ((uint32_t)n > kStaticMaxSegments)
        return fail(TSW_ERR_BUFFER, "tsw_place_segments_static: " + std::to_string(n) + " segments exceed the static scratch limit of " +
                                        std::to_string(kStaticMaxSegments) + "; split the list or use tsw_place_segments");
    if (tile_bytes == 0) tile_bytes = 64u * 1024;
    if ((tile_bytes & 15u) || tile_stride == 0)
        return fail(TSW_ERR_INVALID, "tile size must be a multiple of 16 and stride positive");
    if (pub && pub->done_count && (!pub->table_phys || !pub->table_flag))
        return fail(TSW_ERR_INVALID, "publish block needs both table columns");
    if (n == 0) return TSW_OK;

    StaticDevice& sd = g_static_dev[device];
    std::lock_guard<std::mutex> guard(sd.mu);
    DeviceRestore restore;   // the caller's current device is put back on return
    cudaError_t err = cudaSetDevice(device);
    if (err != cudaSuccess) return fail(TSW_ERR_NO_DEVICE, std::string("cudaSetDevice: ") + cudaGetErrorString(err));
    int rc = static_setup(sd);
    if (rc != TSW_OK) return rc;
    unsigned char* scratch = sd.scratch;

    // Tile numbering.  A segment that does not say how many tiles complete its row is its own row.
    uint64_t t = 0;
    for (int i = 0; i < n; ++i) {
        PlaceDesc& d = sd.host_descs[i];
        memcpy(&d, &segs[i], sizeof(PlaceDesc));
        const uint64_t tiles = (d.bytes + tile_bytes - 1) / tile_bytes;
        sd.host_first[i] = (uint32_t)t;
        t += tiles;
        if (d.row_tiles == 0) {
            d.row_tiles = (uint32_t)tiles;
            d.row_dst = d.dst;
        }
    }
    sd.host_first[n] = (uint32_t)t;
    if (t > 0xffffffffull) return fail(TSW_ERR_INVALID, "too many tiles for one call");

    cudaStream_t s = (cudaStream_t)stream;
    PlaceDesc* d_descs = reinterpret_cast<PlaceDesc*>(scratch);
    uint32_t* d_first = reinterpret_cast<uint32_t*>(scratch + kStaticDescBytes);
    // Pageable source: the runtime has taken its copy when these calls return, so the
    // host-side staging arrays can be reused by the next call.
    err = cudaMemcpyAsync(d_descs, sd.host_descs, sizeof(PlaceDesc) * (size_t)n, cudaMemcpyHostToDevice, s);
    if (err == cudaSuccess)
        err = cudaMemcpyAsync(d_first, sd.host_first, sizeof(uint32_t) * ((size_t)n + 1), cudaMemcpyHostToDevice, s);
    if (err != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("table upload: ") + cudaGetErrorString(err));

    PlaceArgs a;
    memset(&a, 0, sizeof(a));
    a.descs = d_descs;
    a.first_tile = d_first;
    a.n_descs = (uint32_t)n;
    a.tile_bytes = tile_bytes;
    a.tile_lo = tile_first;
    a.tile_hi = (uint32_t)t;
    a.tile_stride = tile_stride;
    a.system_scope = 1;
    a.status = sd.status;
    if (pub) {
        a.done_count = (uint32_t*)pub->done_count;
        a.table_phys = (uint64_t*)pub->table_phys;
        a.table_flag = (uint32_t*)pub->table_flag;
        a.host_phys = (uint64_t*)pub->host_phys;
        a.host_flag = (uint32_t*)pub->host_flag;
        a.flag_value = pub->flag_value;
        a.host_flag_value = pub->flag_value;
        a.ticket = (uint32_t*)pub->ticket;
        a.ticket_chunk = pub->ticket_chunk ? pub->ticket_chunk : 1;
    }
    err = launch_place(a, default_grid_ctas(device), s);
    if (err != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("placement kernel launch: ") + cudaGetErrorString(err));
    return TSW_OK;
}

extern "C" int tsw_place_segments_static_status(int device, void* stream, uint32_t* status, int clear) {
    using namespace tsw;
    if (!status) return fail(TSW_ERR_INVALID, "null argument");
    if (device < 0 || device >= kMaxDevices) return fail(TSW_ERR_INVALID, "device ordinal out of range");
    StaticDevice& sd = g_static_dev[device];
    std::lock_guard<std::mutex> guard(sd.mu);
    DeviceRestore restore;
    cudaError_t err = cudaSetDevice(device);
    if (err != cudaSuccess) return fail(TSW_ERR_NO_DEVICE, std::string("cudaSetDevice: ") + cudaGetErrorString(err));
    int rc = static_setup(sd);
    if (rc != TSW_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    uint32_t word = 0;
    err = cudaMemcpyAsync(&word, sd.status, sizeof(word), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err == cudaSuccess && clear && word) {
        const uint32_t zero = 0;
        err = cudaMemcpyAsync(sd.status, &zero, sizeof(zero), cudaMemcpyHostToDevice, s);
        if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    }
    if (err != cudaSuccess) return fail(TSW_ERR_CUDA, std::string("static status read: ") + cudaGetErrorString(err));
    *status = word;
    return TSW_OK;
}
