/* torpor_swap.h -- C ABI of the B200 swap engine (libtorpor_swap.so).
 *
 * The library replaces one path of Torpor's server: swapping a function's
 * weights between the host model store and the pooled GPU memory manager.
 * In the reference that path is the C++ class server::manager::MemoryManager
 * (include/server/memory_manager.hpp) with its allocator
 * (include/server/block_manager.hpp) and tables (include/server/model_repo.hpp),
 * plus the eviction policy (include/server/evictor.hpp) and the swap decision
 * of the controller (include/server/controller.hpp:296-453).  The reference has
 * no FFI on this path: the executor calls MemoryManager's public methods
 * directly.  Each entry point below therefore stands for one of those methods
 * and cites it; the header-only adapter torpor_b200/adapter/memory_manager.hpp
 * turns them back into the reference's class so src/server compiles unchanged.
 *
 * Conventions: plain pointers and sizes only; every function returns a
 * tsw_status (0 = ok, negative = error) unless stated otherwise; device
 * pointers travel as uint64_t.  Nothing here falls back to the CPU: an engine
 * created on a CUDA device moves bytes only with the library's own sm_100a
 * kernels and fails with TSW_ERR_CUDA / TSW_ERR_NO_DEVICE when it cannot.
 */
#ifndef TORPOR_SWAP_H_
#define TORPOR_SWAP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tsw_engine tsw_engine;
typedef struct tsw_evictor tsw_evictor;
typedef struct tsw_scheduler tsw_scheduler;

typedef enum {
    TSW_OK = 0,
    TSW_ERR_INVALID = -1,         /* bad argument or handle */
    TSW_ERR_NO_DEVICE = -2,       /* data call on a plan-only engine, or no usable CUDA device */
    TSW_ERR_CUDA = -3,            /* a CUDA runtime call failed; see tsw_last_error() */
    TSW_ERR_POOL_EXHAUSTED = -4,  /* the reference exits here (block_manager.hpp:343-352) */
    TSW_ERR_UNKNOWN_MODEL = -5,
    TSW_ERR_TIMEOUT = -6,         /* a bounded wait ran out (the reference blocks forever, memory_manager.hpp:531) */
    TSW_ERR_NOT_FOUND = -7,       /* address is not inside any block of the model */
    TSW_ERR_BUFFER = -8,          /* caller's output buffer is too small */
    TSW_ERR_STATE = -9,           /* call not valid in the current state */
    TSW_ERR_KERNEL = -10          /* a kernel reported an error status */
} tsw_status;

/* Parameter readiness, as in memory_manager.hpp:29-31. */
enum { TSW_READY_HOST = 0, TSW_READY_PINNED = 1, TSW_READY_CUDA = 2 };
/* Model status, as in model_repo.hpp:32-35. */
enum { TSW_MODEL_FULL = 0, TSW_MODEL_INCOMPLETE = 1, TSW_MODEL_PARTIAL = 2, TSW_MODEL_NODATA = 3 };
/* Pool policy: memory_manager.hpp:46-52 (env BLOCK_MANAGER). */
enum { TSW_POOL_BUDDY = 0, TSW_POOL_FIXED = 1 };

typedef struct {
    int device;             /* CUDA device ordinal, or -1 for a plan-only engine: placement and
                               tables are computed, no CUDA call is made and no byte moves */
    int server_id;          /* executor id (MemoryManager::set_server_id, :62-65) */
    int gpu_count;          /* start_trans_thread(gpu_count), :168 */
    uint64_t budget_bytes;  /* MemoryManager(budget), :38-54; 5 GiB are added as the reference does */
    int pool_policy;        /* TSW_POOL_BUDDY | TSW_POOL_FIXED */
    uint64_t host_arena_bytes; /* page-locked host model store carved from one arena of this size;
                               0 = one page-locked allocation per model block */
    const char* host_arena_shm; /* optional POSIX shm name: the arena is created there so that other
                               processes can attach it (tsw_arena_attach) for sharded swaps */
    int grid_ctas;          /* persistent CTAs of the placement kernel; 0 = default (6 per SM; see grid_ctas_host for
                               single-GPU moves with one end in the host store).  A value given here applies to
                               both unless grid_ctas_host is given too */
    int tile_bytes_host;    /* bytes per tile when the source is host memory; 0 = default */
    int tile_bytes_device;  /* bytes per tile when the source is device memory; 0 = default */
    int mover;              /* 0 = tiles moved by loads/stores of the SMs' threads (default); 1 = by the bulk
                               asynchronous copy unit through shared memory where every end is 16-byte
                               aligned (else falls back to 0); 2 = as 0, but on a single-GPU swap-in
                               from the host store the parameters of 4 MiB and more are moved by the
                               copy engine (cudaMemcpyAsync in access order on a second stream, a
                               small kernel behind each rewriting the parameter's table row), for
                               links on which the copy engine reads host memory faster than the SMs
                               do; the write-back of tsw_evict is split the same way.  Env
                               TORPOR_SWAP_MOVER overrides. */
    int shard_static;       /* tsw_swap_in_sharded: 0 = participants draw tiles from a shared counter
                               (default), 1 = tile t is fixed to participant t mod n */
    int host_store_mode;    /* how the host model store is made page-locked (model_repo.hpp:124-141,173-177
                               keeps it pageable): 0 = cudaHostAlloc, portable + device-mapped (default);
                               TSW_STORE_WRITE_COMBINED = the same, write-combined (no CPU-cache snoop on
                               device reads; slow to read back on the CPU); TSW_STORE_HUGE_PAGES = an
                               anonymous mapping (the shm arena when host_arena_shm is set) advised to
                               transparent huge pages, then registered.  Env TORPOR_SWAP_HOST_STORE
                               overrides.  Huge pages apply to the arena only (host_arena_bytes > 0). */
    int ticket_chunk;       /* sharded swaps that draw tiles from the shared counter: tiles taken per
                               draw; 0 = 1 */
    int grid_ctas_host;     /* persistent CTAs of the placement kernel when one end of a single-GPU move is
                               the host store (swap-in from it, write-back into it).  Such a move is bound
                               by PCIe, which a fraction of the SMs saturates, and the CTAs hold their
                               registers for the whole swap: the fewer there are, the more of every SM is
                               left to the function's own kernels that run while its later weights are
                               still arriving (cuda_server.hpp:1265-1268 launches them as soon as their
                               parameters are ready).  0 = default (32).  Env TORPOR_SWAP_GRID_HOST overrides. */
} tsw_config;
enum { TSW_STORE_DEFAULT = 0, TSW_STORE_WRITE_COMBINED = 1, TSW_STORE_HUGE_PAGES = 2 };

void tsw_config_default(tsw_config* cfg);

const char* tsw_last_error(void);       /* thread-local text of the last failure */
const char* tsw_version(void);

/* Process-wide model repository (ModelRepo::getInstance(), model_repo.hpp:67-72). */
int tsw_repo_reset(void);                                        /* forget every model (tests) */
int tsw_repo_add_model_info(const char* func, int gpu);          /* model_repo.hpp:82-85 */
int tsw_repo_remove_model_info(const char* func, int gpu);       /* model_repo.hpp:87-90 */
int tsw_repo_model_status(const char* func, int gpu);            /* DeviceModelInfo::status_, or <0 */
uint64_t tsw_repo_total_size(const char* func);                  /* HostModelInfo::total_size_ */
int tsw_repo_active_devices(const char* func, int* gpus, int cap); /* model_active_device_map_ */

/* Engine life cycle: MemoryManager(budget) + set_server_id + start_trans_thread
 * (memory_manager.hpp:38-65,168-193) / destroy_trans_thread (:229-232). */
int tsw_engine_create(const tsw_config* cfg, tsw_engine** out);
int tsw_engine_destroy(tsw_engine* e);

/* Cold start recorders. */
int tsw_track_begin(tsw_engine* e, const char* func);            /* set_track_model_memory, :67-71 */
int tsw_track_end(tsw_engine* e, const char* func);              /* unset_track_model_memory, :73-80 */
int tsw_malloc(tsw_engine* e, const char* func, uint64_t size, int load_model_flag,
               uint64_t* vptr);                                   /* cudaMallocBackend, :85-94 */
int tsw_free(tsw_engine* e, const char* func, uint64_t vptr);    /* cudaFreeBackend, :97-110 */
/* cudaMemcpyAsyncBackendHtoD with load_model_flag = true (:124-135,141): records the
 * parameter in the host store and uploads it.  stream is a cudaStream_t.  On a plan-only
 * engine (device = -1) payload may be null: address and size are recorded, no byte is kept. */
int tsw_memcpy_h2d_model(tsw_engine* e, const char* func, uint64_t dst_vptr,
                         const void* payload, uint64_t size, void* stream);
int tsw_sync_done(tsw_engine* e, const char* func);              /* init_model_readiness(func), :234-238 */
int tsw_mark_access(tsw_engine* e, uint64_t vptr);               /* try_insert_model_access, :273-284; 1/0 */

/* Forwarded client copies after translation (:112-122,136-163). */
int tsw_memcpy_h2d(tsw_engine* e, const char* func, uint64_t dst_vptr, const void* src, uint64_t size, void* stream);
int tsw_memcpy_d2h(tsw_engine* e, const char* func, void* dst, uint64_t src_vptr, uint64_t size, void* stream);
int tsw_memcpy_d2d(tsw_engine* e, const char* func, uint64_t dst_vptr, uint64_t src_vptr, uint64_t size, void* stream);
int tsw_memset(tsw_engine* e, const char* func, uint64_t vptr, int value, uint64_t size, void* stream);

/* Swap-in: sig_trans_thread(func, src_gpu) (:213-227) = check_and_malloc_model
 * (:451-507) + transfer_model (:331-438).  Returns once blocks are placed, the
 * pointer table is rebound and the placement kernel is enqueued; readiness is
 * published per parameter by the kernel.  src_gpu < 0: from the host store;
 * otherwise from the resident replica of engine `src_gpu` in this process. */
int tsw_swap_in(tsw_engine* e, const char* func, int src_gpu);
/* Sharded swap-in: the tiles of one swap are dealt out to `n_helpers` + 1 engines of
 * this process; every engine reads its share of the host store over its own PCIe
 * link and stores it straight into the target's pool blocks over NVLink.  No
 * counterpart in the reference; the result equals tsw_swap_in(e, func, -1). */
int tsw_swap_in_sharded(tsw_engine* e, const char* func, tsw_engine* const* helpers, int n_helpers);
/* Wait until every accessed parameter of func is on the device (bounded). */
int tsw_wait_ready(tsw_engine* e, const char* func, int64_t timeout_ns);
/* Non-blocking form: the number of accessed parameters still on their way (0 = all there). */
int tsw_poll_ready(tsw_engine* e, const char* func);
int tsw_check_alloc(tsw_engine* e, const char* func);            /* check_model_alloc_status, :195-210; 1/0 */

/* Swap-out: evict_model(func) (:240-259).  The reference moves no bytes; with
 * writeback != 0 the resident parameter bytes are first written back to the
 * host store by the D2H kernel. */
int tsw_evict(tsw_engine* e, const char* func, int writeback);

/* get_cuda_addr (:261-271): client pointer -> current device pointer.  For a
 * model parameter that is being swapped in this waits (at most timeout_ns) for
 * its readiness flag, as check_param_readiness does (:527-540). */
int tsw_translate(tsw_engine* e, const char* func, uint64_t vptr, int search_amid,
                  int64_t timeout_ns, uint64_t* out);
/* Stream-ordered get_cuda_addr: returns the rebound address at once and, when the parameter is
 * still being swapped in, makes `stream` (a cudaStream_t of the same GPU) wait for it with a
 * stream memory operation on the device pointer table -- no host blocking, no device spinning --
 * so the executor can enqueue the kernels of a request before its weights have landed
 * (replaces the blocking wait of cuda_server.hpp:1265-1268 -> memory_manager.hpp:527-540).
 * *waited = 1 if a wait was enqueued.  TSW_ERR_STATE if the parameter is neither resident nor
 * part of a swap in flight (a wait on it could never be satisfied).
 * The wait is bounded from the host.  The word waited on is the row's generation word in
 * host-mapped memory, which the kernel writes when the row completes and which the host can write
 * with a plain store -- no CUDA call, so the release cannot be queued behind the wait it ends (CUDA
 * does not see the ordering a stream memory wait creates; work submitted after it, on any stream,
 * may share its hardware queue).  For the same reason enqueue waits only for swaps whose kernels
 * this process has already launched: after tsw_swap_in / tsw_swap_in_sharded returned, or, with a
 * plan handed to other processes (tsw_swap_plan), after this process's own share was launched.
 * The rows waited for are remembered; they are let go -- the
 * host writes the generation word they wait for, the stream runs on WITHOUT the bytes, and the
 * row is marked failed -- when the whole-model wait gives up (tsw_wait_ready times out or sees a
 * kernel error), when a kernel error is taken note of at the next swap or eviction on the engine,
 * when the model is evicted or its swap-in cannot be placed, when the engine is destroyed, or on
 * request (tsw_release_waiters).  After synchronising a stream that waited, check tsw_poll_ready
 * or tsw_translate: both answer TSW_ERR_KERNEL for a failed row until the model is swapped in
 * again or evicted.  A swap that is repeated (tsw_swap_in after an abandoned plan) releases the
 * waiters of the earlier attempt with the real bytes: generations only grow and a wait is for
 * "at least this generation". */
int tsw_translate_async(tsw_engine* e, const char* func, uint64_t vptr, void* stream, uint64_t* out, int* waited);
/* Let go of every stream still waiting for a parameter of func on this engine (see above);
 * returns how many rows were released without their bytes.  No counterpart in the reference,
 * whose wait (memory_manager.hpp:527-540) has no way out. */
int tsw_release_waiters(tsw_engine* e, const char* func);
int tsw_is_model_address(tsw_engine* e, const char* func, uint64_t vptr);    /* :286-291; 1/0 */
int tsw_valid_memory_address(tsw_engine* e, const char* func, uint64_t vptr); /* :293-298; always 0 */

/* Introspection for parity checks: the tables of model_repo.hpp:37-65 and the readiness
 * map (memory_manager.hpp:33,590) as rows of 64-bit words.
 * blocks (6 words): vaddr, size, is_model, in_cuda, cuda_addr, in_pin(=0), in the order
 *   swap-in requests pool blocks; params (7 words): vaddr, size, block_vaddr, cuda_addr,
 *   readiness_flag, readiness_addr, accessed -- access order first, then the rest by vaddr.
 * canonical != 0 rewrites every address into the canonical address space (pool base ->
 * fixed base), which makes the tables of two runs comparable word for word.
 * Both return the number of rows (also when out == NULL). */
int tsw_dump_blocks(tsw_engine* e, const char* func, int canonical, uint64_t* out, int cap);
int tsw_dump_params(tsw_engine* e, const char* func, int canonical, uint64_t* out, int cap);
/* Pool geometry: base of the pool, number of 128 MiB chunks, and the canonical base that
 * addresses are keyed by internally (so that table order does not depend on where the
 * driver happened to map the pool). */
int tsw_pool_info(tsw_engine* e, uint64_t* pool_base, uint64_t* n_chunks, uint64_t* canon_base);
/* The canonical form of one address: inside a block the pool has handed out, else inside a
 * block of `func` as the client knows it; any other value comes back unchanged. */
int tsw_canonical_address(tsw_engine* e, const char* func, uint64_t addr, uint64_t* out);
int tsw_read_phys(tsw_engine* e, uint64_t addr, void* out, uint64_t size);
int tsw_read_host_store(tsw_engine* e, const char* func, uint64_t vptr, void* out, uint64_t size);
/* Per-parameter 2 x 64-bit checksum of the RESIDENT bytes, computed on the device
 * (s1 = sum of 32-bit words, s2 = sum of (index+1)*word, both mod 2^64; a ragged tail is
 * zero-extended).  out holds 2 words per parameter in tsw_dump_params order. */
int tsw_checksum_resident(tsw_engine* e, const char* func, uint64_t* out, int cap);

/* The data mover on its own: copy `n` segments with the placement kernel on this engine's
 * transfer stream.  Addresses are device-visible: page-locked host memory, this GPU's memory
 * or a peer's (peer access or an opened IPC handle).  Tiles of `tile_bytes` are numbered over
 * the whole list; this call moves tiles tile_first, tile_first + tile_stride, ... below
 * tile_end (0 = to the end of the list), so that several engines -- in one process or one per process -- can share a list.  With `pub`, the
 * kernel counts finished tiles per table row in done_count (zeroed memory on the target GPU,
 * shared by all participants) and whoever finishes the last tile of a row writes row_dst and
 * flag_value into that row of the table columns.  This is the building block of
 * tsw_swap_in_sharded and of multi-process sharded swaps; it has no counterpart in the
 * reference, whose mover is cudaMemcpyAsync per parameter (memory_manager.hpp:389-396). */
typedef struct {
    uint64_t src, dst, bytes;
    uint64_t row_dst;    /* address published for the row; used when row_tiles != 0 */
    uint32_t row;        /* row of the table this segment contributes to */
    uint32_t row_tiles;  /* tiles that complete the row over all segments and participants;
                            0 = count the tiles of this row in this list, publish the first dst */
} tsw_segment;
typedef struct {
    uint64_t done_count;   /* uint32 per row, device memory of the target, zero before the swap */
    uint64_t table_phys;   /* uint64 per row, device memory of the target */
    uint64_t table_flag;   /* uint32 per row, device memory of the target */
    uint64_t host_phys;    /* optional host-mapped mirrors of the two columns (0 = none) */
    uint64_t host_flag;
    uint32_t flag_value;
    uint32_t ticket_chunk; /* tiles drawn per ticket (0 = 1) */
    uint64_t ticket;       /* optional: uint32 on the target, set to tile_first before the swap.  When
                              given, tile_stride is ignored and the CTAs of every participant draw
                              their tiles from this counter, so faster links move more tiles */
} tsw_publish;
int tsw_place_segments(tsw_engine* e, const tsw_segment* segs, int n, uint32_t tile_bytes, uint32_t tile_first,
                       uint32_t tile_stride, uint32_t tile_end, const tsw_publish* pub, int sync);

/* One process per GPU.  A swap-in can be carried out by several processes, each driving the
 * placement kernel on its own GPU (tsw_place_segments with a tile stride): the target process
 * places and rebinds with tsw_swap_plan, which returns the moves (addresses valid in the target
 * process) instead of launching them; the others reach the target's pool and table through
 * CUDA IPC (tsw_ipc_regions on the target, tsw_ipc_open elsewhere) and the host store through
 * a shared-memory arena (config host_arena_shm on the target, tsw_arena_attach elsewhere), and
 * rebase the addresses accordingly; when all are done the target calls tsw_swap_commit, which
 * takes the rows the kernels published on the device over into its host-visible table.
 * If a participant went away, tsw_swap_commit returns TSW_ERR_STATE and keeps the unfinished rows
 * listed: commit again later, or call tsw_swap_in, which moves what is missing by itself (the tile
 * counters of the abandoned rows are cleared first).
 * No counterpart in the reference (one process, one GPU per swap). */
typedef struct {
    uint64_t base, size;
    unsigned char handle[64];   /* cudaIpcMemHandle_t */
} tsw_ipc_region;
int tsw_swap_plan(tsw_engine* e, const char* func, tsw_segment* segs, int cap, uint32_t* tile_bytes, tsw_publish* pub);
int tsw_swap_commit(tsw_engine* e, const char* func);
int tsw_ipc_regions(tsw_engine* e, tsw_ipc_region* out, int cap);   /* returns the number of regions */
int tsw_ipc_open(tsw_engine* e, const void* handle, uint64_t* mapped_base);
/* What the CUDA driver knows about an address in this process (cudaPointerGetAttributes):
 * type 0 = unknown to the driver, 1 = page-locked host, 2 = device, 3 = managed. */
int tsw_pointer_info(tsw_engine* e, uint64_t addr, int* type, int* device, uint64_t* device_pointer, uint64_t* host_pointer);
int tsw_arena_info(tsw_engine* e, uint64_t* host_base, uint64_t* dev_base, uint64_t* size, uint64_t* used);
int tsw_arena_attach(tsw_engine* e, const char* shm_name, uint64_t size, uint64_t* dev_base);

/* tsw_place_segments in two pipelined steps, for a helper whose link the copy engine reads faster than
 * the SMs do: each chunk of `chunk_tiles` tiles (0 = 64 MiB worth) of the range [tile_first, tile_end) is
 * brought from its host source into this engine's GPU by cudaMemcpyAsync on a second stream, then stored
 * to its destination and counted by the placement kernel while the next chunk is being fetched.  Tiles
 * are dealt by range, not drawn (pub->ticket is ignored).  The engine keeps a staging area of the size
 * of the largest range it was given.  No counterpart in the reference. */
int tsw_place_segments_pipelined(tsw_engine* e, const tsw_segment* segs, int n, uint32_t tile_bytes, uint32_t tile_first,
                                 uint32_t tile_end, const tsw_publish* pub, uint32_t chunk_tiles, int sync);

/* tsw_place_segments for callers that must not allocate.  No counterpart in the reference.
 *
 * Meant for code on the steady-state swap path of a GPU-sharing server -- an executor that
 * forwards intercepted client CUDA calls, a plugin in a process whose device memory already
 * belongs to the block pool, a helper that only lends its PCIe link to a sharded swap --
 * where a device allocation would synchronise the GPU under the running inference kernels,
 * could fail because the pool owns the memory, or would be intercepted itself.  It needs no
 * engine: it takes the device ordinal and a cudaStream_t, and calls neither cudaMalloc nor
 * cudaFree nor any allocating routine.  The descriptor table the kernel reads lives in a
 * fixed 1 MiB array inside the loaded module (so every GPU that uses the library gives up
 * 1 MiB until the process exits), which limits one call to 16384 segments; more are refused
 * with TSW_ERR_BUFFER.  All calls on a device share that array: calls whose GPU work overlaps
 * (different streams or threads) corrupt each other's table -- issue them on one stream or
 * serialise them.  The array's device address is looked up during the first call made for a
 * device; make that first call outside of any stream capture.
 * Differences from tsw_place_segments: a segment with row_tiles == 0 completes its own row
 * (rows are not summed over the list), and no device timing is recorded. */
int tsw_place_segments_static(int device, const tsw_segment* segs, int n, uint32_t tile_bytes, uint32_t tile_first,
                              uint32_t tile_stride, const tsw_publish* pub, void* stream);
/* The word in which the kernel of tsw_place_segments_static reports a table that does not fit its
 * tile numbering -- what overlapping calls on one device produce -- read back after `stream` has
 * drained (this call synchronises it); 0 = nothing reported.  clear != 0 resets a non-zero word.
 * Allocates nothing either.  The cached array addresses do not survive a cudaDeviceReset; the
 * caller's current device is unchanged by both calls.  No counterpart in the reference. */
int tsw_place_segments_static_status(int device, void* stream, uint32_t* status, int clear);

/* Counters: kernels launched by this engine, bytes they were asked to move, and device
 * time of the last swap on the transfer stream (CUDA events), in nanoseconds. */
int tsw_stats(tsw_engine* e, uint64_t* kernel_launches, uint64_t* bytes_moved, uint64_t* last_swap_device_ns);

/* Eviction policy: Evictor / LRUEvictor / InterferenceAwareEvictor (evictor.hpp:14-264).
 * kind: "LRU" or "IA".  check_and_add returns the number of victims and writes their names
 * '\n'-joined; unlike the reference it returns TSW_ERR_STATE instead of spinning when
 * nothing can be evicted (evictor.hpp:211-224). */
int tsw_evictor_create(const char* kind, int gpu_count, uint64_t budget, tsw_evictor** out);
int tsw_evictor_destroy(tsw_evictor* ev);
int tsw_evictor_check_and_add(tsw_evictor* ev, int gpu, const char* func, uint64_t size, int level,
                              char* victims, int cap);
int tsw_evictor_force_evict(tsw_evictor* ev, int gpu, const char* func);
int tsw_evictor_lock(tsw_evictor* ev, int gpu, const char* func);
int tsw_evictor_unlock(tsw_evictor* ev, int gpu, const char* func);

/* Swap scheduler: the decision functions of the controller (controller.hpp:296-389) for any
 * number of GPUs.  policy: "IA" (interference-aware, default) or "RAND".  pcie_pairs[i] = the
 * GPU sharing GPU i's PCIe uplink and nvlink[i*n+j] in {-1,0,1,2} replace the reference's
 * hard-coded 4-GPU tables (:116-118); NULL = NVSwitch defaults (all peers fast, sibling i^1).
 * status values are the reference's ExecutorStatus_* (-1 available ... 5 cold start, :18-24).
 * tsw_sched_decide answers gpu = -1 when no GPU is available (the caller queues the request);
 * src_gpu >= 0 asks for a replica swap from that GPU; it reads the replicas of `func` from the
 * process-wide repository (tsw_repo_add_model_info / tsw_repo_remove_model_info). */
/* Fill the two tables from the machine: peer-access attributes for nvlink, PCI paths for pairs. */
int tsw_topology_discover(int gpu_count, int* pcie_pairs, int* nvlink);
int tsw_sched_create(int gpu_count, const char* policy, const int* pcie_pairs, const int* nvlink, tsw_scheduler** out);
int tsw_sched_destroy(tsw_scheduler* s);
int tsw_sched_set_status(tsw_scheduler* s, int gpu, int status);
int tsw_sched_set_level(tsw_scheduler* s, const char* func, int level);
int tsw_sched_decide(tsw_scheduler* s, const char* func, int* gpu, int* src_gpu, int* status);
/* 1-link or k-link swap-in: the GPUs that can lend their PCIe link to a swap-in of `dst` from the
 * host store right now (helpers for tsw_swap_in_sharded); returns their number.  Read from the same
 * occupancy signal the reference's scheduler uses to pick a GPU (status RunPcie* / RunColdStart =
 * link busy, :379-385): available GPUs (with include_running, also GPUs that run in place or swap
 * over NVLink), minus those whose uplink sibling (pcie_pairs) is dst, is loading, or already lends.
 * No reference counterpart: the reference always uses one link per swap. */
int tsw_sched_helpers(tsw_scheduler* s, int dst, int include_running, int* helpers, int cap);

/* Request handling around a swap: what the controller does with each router request and each
 * executor completion (controller.hpp:130-262) on top of the scheduler and the eviction
 * policy above -- round-robin placement of cold starts (:283-294), one request per GPU with a
 * FIFO for the rest (:176-178,242-262), check_eviction (:392-400), send_exec_req (:402-418),
 * send_load_req (:420-427) and the pin on a source replica while a GPU copies from it
 * (:442-453).  No sockets and no executor threads: every signal the reference would send to
 * an executor (`signal` = ExecutorSignal_* of utils.hpp:70-74; a load is 4 + 1 + src_gpu, so
 * 4 means "from the host store") and every acknowledgement it would return to the router
 * (`resp` = the GPU chosen, or -1) goes to a callback, in the reference's order.  Replicas and
 * model sizes are read from and written to the process-wide repository, as the reference's
 * controller does with the ModelRepo singleton.
 * type: TSW_REQ_* (RequestType of proto/signal.proto); payload: the model level "0".."2" for
 * TSW_REQ_EXECUTE_AFTER_LOAD, an optional GPU index for TSW_REQ_EXECUTE / TSW_REQ_UNLOAD.
 * Where the reference would spin because nothing can be evicted (evictor.hpp:84-95,211-224):
 * if pinned replicas are in the way, the request waits in the queue like one that found every
 * GPU busy (TSW_OK, nothing sent, no acknowledgement yet) and is tried again at the next
 * completion; a model at or above the limit can never fit, and the call returns TSW_ERR_STATE,
 * sends nothing and drops the request.  A cold start that has finished is entered even if its
 * GPU stays over the limit (it is there already); whatever is not pinned is unloaded for it.
 * A controller, a scheduler and an eviction policy are each driven from one thread, as the
 * reference's controller loop drives them; they take no lock of their own. */
typedef struct tsw_controller tsw_controller;
typedef void (*tsw_signal_fn)(void* user, int gpu, int signal, const char* func);
typedef void (*tsw_ack_fn)(void* user, int ack, int resp);
#define TSW_REQ_EXECUTE_AFTER_LOAD 0
#define TSW_REQ_EXECUTE 1
#define TSW_REQ_LOAD 2
#define TSW_REQ_UNLOAD 3
#define TSW_SIGNAL_NOTIFY 0
#define TSW_SIGNAL_STARTUP 1
#define TSW_SIGNAL_EXECUTE 2
#define TSW_SIGNAL_UNLOAD 3
#define TSW_SIGNAL_LOAD 4
int tsw_ctrl_create(int gpu_count, uint64_t mem_limit_bytes, const char* schedule_policy, const char* evict_policy,
                    const int* pcie_pairs, const int* nvlink, tsw_signal_fn on_signal, tsw_ack_fn on_ack, void* user,
                    tsw_controller** out);
int tsw_ctrl_destroy(tsw_controller* c);
int tsw_ctrl_request(tsw_controller* c, int type, const char* func, const char* payload);
int tsw_ctrl_complete(tsw_controller* c, int executor);    /* the executor's "done" on controller_sync_queue */
int tsw_ctrl_executor_status(tsw_controller* c, int gpu, int* status, char* func, int cap);
int tsw_ctrl_queue_depth(tsw_controller* c);
int tsw_ctrl_helpers(tsw_controller* c, int dst, int include_running, int* helpers, int cap);  /* tsw_sched_helpers on its scheduler */

#ifdef __cplusplus
}
#endif
#endif /* TORPOR_SWAP_H_ */
