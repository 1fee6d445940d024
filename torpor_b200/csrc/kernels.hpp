// Launch interface of the sm_100a kernels (kernels.cu).
#ifndef TORPOR_SWAP_KERNELS_HPP_
#define TORPOR_SWAP_KERNELS_HPP_

#include <cstdint>
#include <cuda_runtime.h>

namespace tsw {

// One parameter's move.  Tiles are numbered over the whole swap: parameter k
// owns tiles [first_tile[k], first_tile[k+1]).
struct PlaceDesc {
    uint64_t src;       // host-mapped, local or peer address
    uint64_t dst;       // local pool, peer pool or host-mapped address
    uint64_t bytes;
    uint64_t row_dst;   // address published for the row (start of the whole parameter)
    uint32_t row;       // row of the pointer table this move contributes to
    uint32_t row_tiles; // tiles of that row over ALL segments and participants
};

struct PlaceArgs {
    const PlaceDesc* descs;       // device-readable, n_descs entries
    const uint32_t* first_tile;   // device-readable, n_descs + 1 entries
    uint32_t n_descs;
    uint32_t tile_bytes;          // multiple of 16
    uint32_t tile_lo, tile_hi;    // this launch handles tiles tile_lo + i * tile_stride < tile_hi
    uint32_t tile_stride;
    // Completion and rebind.  done_count lives with the TARGET of the swap so that
    // several GPUs can finish tiles of the same parameter; may be null (then nothing
    // is published and the launch is just a copy).
    uint32_t* done_count;         // per row, must be 0 at launch, left 0 on completion
    uint64_t* table_phys;         // device pointer table: rebound address per param
    uint32_t* table_flag;         //                       readiness per param
    uint64_t* host_phys;          // host-mapped mirror of the two columns (may be null)
    uint32_t* host_flag;
    uint32_t* host_gen;           // host-mapped generation word per param: what stream-ordered waits wait on (may be null)
    uint32_t flag_value;          // written to the device flag column when a param completes
    uint32_t host_flag_value;     // written to the host-mapped flag column
    uint32_t system_scope;        // 1: stores may target a peer GPU / host memory
    // Dynamic dealing: when set, CTAs of every participating GPU draw the next `ticket_chunk`
    // tiles from this counter (on the target GPU) instead of a fixed stride, so that a GPU
    // with a faster path to the host store ends up moving more of the tiles.
    uint32_t* ticket;
    uint32_t ticket_chunk;
    uint32_t* status;             // device word, set non-zero on an internal inconsistency
    // Segments of at least this many bytes are left alone by this launch (0 = none): the copy engine
    // moves them, and publish_rows rewrites their table rows behind each copy.
    uint64_t skip_min_bytes;
};

// Descriptor-driven placement copy: host store -> pool blocks (swap-in), pool ->
// pool across NVLink (replica swap / gather), pool -> host store (write-back).
// mover: 0 = loads and stores by the SMs' threads (place_kernel), 1 = the bulk asynchronous copy
// unit through shared memory (place_kernel_bulk; needs 16-byte aligned sources and destinations).
cudaError_t launch_place(const PlaceArgs& a, int grid_ctas, cudaStream_t stream, int mover = 0);

// Rewrite the table rows of segments [lo, hi) of a.descs as the placement kernel does for a
// completed parameter (device table, host-mapped mirror, generation word): the publish step on
// its own, for parameters whose bytes a copy engine moved earlier in the same stream.
cudaError_t launch_publish_rows(const PlaceArgs& a, uint32_t lo, uint32_t hi, cudaStream_t stream);

// Per-parameter checksums of device-resident bytes; out has 2 words per row and must be
// zeroed by the caller.
struct SumDesc {
    uint64_t addr;
    uint64_t bytes;
    uint32_t first_tile;
    uint32_t row;
};
cudaError_t launch_checksum(const SumDesc* descs, uint32_t n_descs, uint32_t total_tiles, uint32_t tile_bytes,
                            unsigned long long* out, int grid_ctas, cudaStream_t stream);

int default_grid_ctas(int device);
int default_grid_ctas_host(int device);   // for moves with one end in host memory

}  // namespace tsw
#endif
