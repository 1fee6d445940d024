/* TEST INFRASTRUCTURE ONLY -- the scenario ABI of the swap-path checkers.
 *
 * Two shared objects export exactly this interface:
 *   oracle/_ref/libtorpor_ref_fake.so / libtorpor_ref_cuda.so
 *       the reference's own headers compiled where they lie (ref_harness.cpp)
 *   oracle/libtorpor_oracle.so
 *       the CPU restatement of the same algorithm (torpor_oracle.cpp)
 * so that one test driver can replay a scenario against either and compare the
 * normalised results with the shipped engine.  Only tests, the smoke check and
 * the benchmark's CPU-baseline / reference legs may load them.
 *
 * A scenario is the call stream a Torpor executor makes into its memory
 * manager (include/server/cuda_server.hpp:223-253,951-978,1027-1037):
 *   track_begin -> malloc* -> memcpy_h2d_model* -> sync_done -> malloc*(non-model)
 *   -> mark_access* -> track_end -> { evict | swap_in + wait_ready }*
 */
#ifndef TORPOR_TSO_ABI_H_
#define TORPOR_TSO_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Forget every model, manager and fake device address handed out so far. */
void tso_reset_world(void);

/* One memory manager per GPU (include/server/memory_manager.hpp:38-54,62-65,168-193).
 * block_manager: "Buddy" (default) or "Fixed".  buffer_size: bytes per readiness
 * group (reference default 2 MiB).  io_threads: pageable->pinned staging threads. */
void* tso_create(int server_id, uint64_t budget_bytes, int gpu_count,
                 const char* block_manager, uint64_t buffer_size, int io_threads);
void tso_destroy(void* h);

void tso_track_begin(void* h, const char* func);                 /* :67-71   */
uint64_t tso_malloc(void* h, const char* func, uint64_t size, int load_model_flag); /* :85-94 */
void tso_free(void* h, const char* func, uint64_t vptr);         /* :97-110  */
int tso_memcpy_h2d_model(void* h, const char* func, uint64_t dst,
                         const void* payload, uint64_t size);    /* :124-142 */
void tso_sync_done(void* h, const char* func);                   /* :234-238 via cuda_server.hpp:951-962 */
int tso_mark_access(void* h, uint64_t vptr);                     /* :273-284 */
void tso_track_end(void* h, const char* func);                   /* :73-80   */

void tso_swap_in(void* h, const char* func, int src_gpu);        /* :213-227 */
/* Blocks until the last parameter in access order is on the device, then
 * until the staging blocks are recycled.  Returns microseconds spent waiting
 * for readiness only. */
int64_t tso_wait_ready(void* h, const char* func);
/* swap_in + wait for readiness; returns microseconds from the signal to the
 * last parameter being published (what the reference logs at :352,:413). */
int64_t tso_swap_in_timed(void* h, const char* func, int src_gpu);
/* reference headers only: the pageable -> pinned pack by the I/O threads alone (:311-329), microseconds */
int64_t tso_pack_timed(void* h, const char* func);
void tso_evict(void* h, const char* func);                       /* :240-259 */
uint64_t tso_translate(void* h, const char* func, uint64_t vptr); /* :261-271 */
int tso_check_alloc(void* h, const char* func);                  /* :195-210 */
int tso_is_model_address(void* h, const char* func, uint64_t vptr); /* :286-291 */

/* Controller-side status bits (include/server/model_repo.hpp:82-90). */
void tso_set_model_status(const char* func, int gpu, int full);
uint64_t tso_total_size(const char* func);

/* Pool geometry: chunk base addresses in allocation order. */
int tso_pool_chunks(void* h, uint64_t* out, int cap);

/* Tables.  Blocks come in the iteration order of the model's block map (the
 * order in which swap-in requests pool blocks), 6 words each:
 *   vaddr, size, is_model, in_cuda, cuda_addr, in_pin.
 * Params come in first-run access order followed by never-accessed params in
 * ascending vaddr, 7 words each:
 *   vaddr, size, block_vaddr, cuda_addr, readiness_flag, readiness_addr, accessed. */
int tso_dump_blocks(void* h, const char* func, uint64_t* out, int cap);
int tso_dump_params(void* h, const char* func, uint64_t* out, int cap);

/* Bytes at a physical ("device") address, and the authoritative host copy. */
int tso_read_phys(void* h, uint64_t addr, void* out, uint64_t size);
int tso_read_host_store(void* h, const char* func, uint64_t vptr, void* out, uint64_t size);

/* Eviction policy (include/server/evictor.hpp).  kind: "LRU" or "IA".
 * check_and_add writes the victims as a '\n'-joined list and returns their
 * number, or -1 if the buffer is too small. */
void* tso_evictor_create(const char* kind, int gpu_count, uint64_t budget);
void tso_evictor_destroy(void* e);
int tso_evictor_check_and_add(void* e, int gpu, const char* func, uint64_t size, int level,
                              char* victims, int cap);
void tso_evictor_force_evict(void* e, int gpu, const char* func);
void tso_evictor_lock(void* e, int gpu, const char* func);
void tso_evictor_unlock(void* e, int gpu, const char* func);

/* All-pairs peer access as the controller enables it at start-up (controller.hpp:63-75); returns the
 * number of directed pairs enabled (0 without real devices). */
int tso_enable_peer_access(int gpu_count);

/* Swap decision of the controller (include/server/controller.hpp:296-389).  The reference
 * checker answers with the reference's own Controller object (controller.hpp compiled where
 * it lies, zmq / executor headers shadowed) and only accepts the 4-GPU tables hard-coded there
 * (:116-118), returning NULL otherwise; the restatement takes any tables.
 * out3 = { gpu, src_gpu, status }; replicas are read from tso_set_model_status. */
void* tso_sched_create(int n, const char* policy, const int* pcie_pairs, const int* nvlink);
void tso_sched_destroy(void* s);
void tso_sched_set_status(void* s, int gpu, int status);
void tso_sched_set_level(void* s, const char* func, int level);
void tso_sched_decide(void* s, const char* func, int* out3);

/* The controller's handling of one router request or one executor completion
 * (include/server/controller.hpp:130-262).  The reference checker runs the reference's own loop
 * for exactly one event on its Controller object (the socket stand-in feeds the event and ends
 * the loop); it accepts 4 GPUs with the tables of :116-118 and a whole number of GiB below 25
 * (MEM_LIMIT_IN_GB, :84-91), else NULL.  `trace` receives what was sent while handling the
 * event, one line each, in order: "S <gpu> <signal> <func>" for a signal to an executor and
 * "A <ack> <resp>" for the acknowledgement to the router; the return value is the size the text
 * needs including its terminator.  Model sizes and replicas are those of the checker's
 * repository (tso_malloc under tso_track_begin; tso_set_model_status).  Function names must not
 * contain blanks. */
void* tso_ctrl_create(int n, uint64_t mem_limit_bytes, const char* sched_policy, const char* evict_policy,
                      const int* pcie_pairs, const int* nvlink);
void tso_ctrl_destroy(void* c);
int tso_ctrl_request(void* c, int type, const char* func, const char* payload, char* trace, int cap);
int tso_ctrl_complete(void* c, int executor, char* trace, int cap);

/* The reference's executor (include/server/cuda_server.hpp), exported by libtorpor_ref_exec.so only.
 * tso_exec_create builds a CUDAExecutor on the fake GPU `id` and runs its loop (cuda_server.hpp:99-262)
 * on a thread; tso_exec_signal is what the controller does to it (controller.hpp:429-431), and
 * tso_exec_queries hands it one serialised QueryList as a client's sender would, returning what it
 * sent back (records of a 4-byte little-endian length + serialised response; the return value is the
 * size the records need).  Kernels are looked up by name in a table the caller fills
 * (tso_exec_register_kernel; the reference fills it from the fat binaries it links); a launch is
 * recorded, not run: tso_exec_launches returns one line per launch, the kernel's name and each
 * argument's bytes in hex as the executor passed them to cudaLaunchKernel.  tso_exec_manager is the
 * executor's own MemoryManager as a handle for the tso_dump_* / tso_wait_ready calls above (never
 * pass it to tso_destroy).  tso_exec_completions drains controller_sync_queue. */
void tso_exec_register_kernel(const char* name);
void* tso_exec_create(int id, uint64_t budget_bytes, int gpu_count);
void* tso_exec_manager(void* exec);
void tso_exec_destroy(void* exec);
void tso_exec_signal(void* exec, int signal, const char* func);
int tso_exec_queries(void* exec, const void* query_list, int n, void* out, int cap);
int tso_exec_launches(char* out, int cap);
int tso_exec_completions(int* out, int cap);
void tso_exec_reset(void);

const char* tso_impl_name(void);

#ifdef __cplusplus
}
#endif
#endif
