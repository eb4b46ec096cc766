/*
 * b200sort - C ABI of the B200 (sm_100a) SORT task kernels.
 *
 * This is the boundary a Legate task body binds instead of the reference's
 * CUB/Thrust/NCCL calls.  Plain C types only; `void*` stands for
 * `cudaStream_t` and `ncclComm_t` so the header needs no CUDA/NCCL include.
 * All device pointers are CUDA device addresses on the current device.
 *
 * Conventions
 *   - every function returns a b2s_status_t and never aborts or throws; the
 *     caller decides (the reference aborts the process on CUDA/NCCL errors,
 *     src/cupynumeric/cuda_help.h:238-300);
 *   - no function allocates device memory: scratch is a caller-provided
 *     workspace (b2s_workspace_bytes) or comes from the caller's allocator
 *     callback (b2s_dist_sort_1d), because in the reference every buffer has
 *     to come from the task's Legate pool (src/cupynumeric/sort/sort.h:94-113,
 *     with_has_allocations);
 *   - work is enqueued on the given stream; local sorts return without
 *     synchronising;
 *   - the sort is always stable, whatever `stable` says (the reference's radix
 *     path ignores the flag too, src/cupynumeric/sort/sort.cu:63-81); floats sort
 *     as -inf < ... < -0.0 == +0.0 < ... < +inf < NaN with the input's bit
 *     patterns preserved; complex keys sort by (real, imaginary), each part
 *     ordered like a float (complex64 keys must be 8-byte aligned).
 */
#ifndef B200SORT_H_
#define B200SORT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  B2S_OK              = 0,
  B2S_ERR_INVALID_ARG = 1,
  B2S_ERR_CUDA        = 2,
  B2S_ERR_NCCL        = 3,
  B2S_ERR_WORKSPACE   = 4, /* workspace too small or misaligned */
  B2S_ERR_TIMEOUT     = 5, /* a bounded device-side wait ran out */
  B2S_ERR_UNSUPPORTED = 6
} b2s_status_t;

/* Element types of the SORT task's input store; one per dtype the Python layer can send
 * (cupynumeric/_utils/array.py:29-44).  The task layer maps legate::Type::Code to these. */
typedef enum {
  B2S_BOOL       = 1,
  B2S_INT8       = 2,
  B2S_INT16      = 3,
  B2S_INT32      = 4,
  B2S_INT64      = 5,
  B2S_UINT8      = 6,
  B2S_UINT16     = 7,
  B2S_UINT32     = 8,
  B2S_UINT64     = 9,
  B2S_FLOAT16    = 10,
  B2S_FLOAT32    = 11,
  B2S_FLOAT64    = 12,
  B2S_COMPLEX64  = 13,
  B2S_COMPLEX128 = 14
} b2s_dtype_t;

/* Human-readable name of a status code.  (Role of the messages printed by check_cuda /
 * check_nccl, src/cupynumeric/cuda_help.h:238-250.) */
const char* b2s_status_string(int status);

/* Library version, major*10000 + minor*100 + patch. */
int b2s_version(void);

/* Bytes of device scratch b2s_local_sort needs for this problem.  Replaces CUB's
 * "query temp_storage_bytes with a null pointer" calls
 * (src/cupynumeric/sort/cub_sort.cuh:60-64,84-92,120-131,153-167). */
int b2s_workspace_bytes(int dtype, size_t volume, size_t segment, int argsort, size_t* bytes);

/* Sorts a dense row-major tile along its last axis: `volume` elements made of
 * `volume / segment` independent segments of `segment` elements.
 *
 *   keys_in   input elements (never written unless keys_out == keys_in)
 *   keys_out  sorted elements; may be NULL when idx_out != NULL; may equal keys_in
 *   idx_out   NULL for sort; for argsort receives int64 positions along the sort axis:
 *             1-D (ndim_is_1 != 0): index_offset + i ;  N-D: i % segment + index_offset
 *             (src/cupynumeric/sort/sort.cu:1851-1862, sort.h:83-92)
 *   ws        device scratch of at least b2s_workspace_bytes(...) bytes, 256-byte aligned
 *
 * Replaces local_sort<CODE> -> cub_local_sort / thrust_local_sort
 * (src/cupynumeric/sort/sort.cu:63-96, cub_sort.cuh:36-193, thrust_sort.cuh:37-124) together
 * with the index initialisation thrust::sequence / thrust::transform (sort.cu:1851-1862).
 * A device-side wait that ran out is reported by b2s_check_status on the same workspace. */
int b2s_local_sort(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                   size_t segment, int64_t index_offset, int ndim_is_1, int stable, void* ws,
                   size_t ws_bytes, void* cuda_stream);

/* Synchronises the stream and reports the device-side status word of the last b2s_local_sort
 * that used this workspace (B2S_OK or B2S_ERR_TIMEOUT).  Stands where the reference has
 * CUPYNUMERIC_CHECK_CUDA_STREAM (src/cupynumeric/cuda_help.h:291-302). */
int b2s_check_status(void* ws, void* cuda_stream);

/* Self-test of the bounded device-side waits: runs a small sort of the library's own whose first
 * tile is deliberately never processed, with a poll limit of a few thousand, so that the waits on
 * that tile run out within milliseconds.  Afterwards b2s_check_status(ws, stream) must answer
 * B2S_ERR_TIMEOUT, and the workspace, the stream and the context must still be usable.  Nothing
 * traps, faults or waits without a bound.  `ws`: at least 2 MiB, 256-byte aligned.  (The reference
 * has no bounded waits to test: its library kernels are not its own.) */
int b2s_selftest_wait_timeout(void* ws, size_t ws_bytes, void* cuda_stream);

/* Same contract as b2s_local_sort, for callers that cannot hand over a workspace because they
 * cannot allocate one: for instance a task body under a runtime that forbids cudaMalloc while
 * tasks are in flight, or a thread whose memory pool is exhausted.  It has no counterpart in the
 * reference.  The scratch is a fixed device array of B2S_NOALLOC_SCRATCH_BYTES that each GPU
 * holds from the moment the library is loaded; the call allocates nothing and returns
 * B2S_ERR_WORKSPACE when b2s_workspace_bytes(...) for the problem exceeds that size.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before any stream capture begins.  All calls on a device share the one array:
 * two calls whose kernels may overlap on the GPU (different streams, no ordering) race with each
 * other; calls on one stream are safe.  A device-side wait that ran out is read back with
 * b2s_noalloc_check_status (the status word lives in the same array, so it reports the last call
 * made on the current device). */
#define B2S_NOALLOC_SCRATCH_BYTES (32u << 20)
int b2s_local_sort_noalloc(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                           size_t segment, int64_t index_offset, int ndim_is_1, void* cuda_stream);
/* b2s_check_status for the fixed scratch of b2s_local_sort_noalloc on the current device.  Like
 * that entry point it allocates nothing and has no counterpart in the reference. */
int b2s_noalloc_check_status(void* cuda_stream);

/* ---- distributed 1-D sort ------------------------------------------------------------------- */

/* Device memory from the caller's pool, 256-byte aligned, valid on the current device; NULL on
 * failure.  Role of legate::create_buffer<T>(n, Memory::GPU_FB_MEM) in the reference
 * (src/cupynumeric/sort/sort.cu:1833-1869). */
typedef void* (*b2s_alloc_fn)(void* ctx, size_t bytes);
/* Returns memory obtained from the paired b2s_alloc_fn (Buffer::destroy(), sort.cu:1933-1936). */
typedef void (*b2s_free_fn)(void* ctx, void* ptr);
/* Optional host barrier among the point tasks of one launch, called around every NCCL call
 * like context.concurrent_task_barrier() (sort.cu:1313-1315,1393,1412,1511,1530,1686,1734).
 * May be NULL when each rank is a process of its own. */
typedef void (*b2s_barrier_fn)(void* ctx);

/* The collectives the distributed calls need, supplied by the host runtime.  All buffers are
 * device memory of the calling rank; every rank of the group makes the same call with the same
 * sizes, on its own stream.  Each function returns a b2s_status_t.
 *   all_gather  every rank contributes `bytes` from `send` and receives the nranks contributions,
 *               in rank order, in `recv`
 *   barrier     completes on a rank's stream only after every rank has enqueued it behind its
 *               earlier work on that stream
 *   exchange    grouped point-to-point transfers: send send_bytes[p] bytes from send_ptr[p] to
 *               rank p and receive recv_bytes[p] bytes from it into recv_ptr[p] (arrays of nranks
 *               entries; the caller's own entry is ignored; zero sizes are skipped)
 * In the reference these are ncclAllGather / grouped ncclSend+ncclRecv on the communicator Legate
 * hands the task (src/cupynumeric/sort/sort.cu:1387-1413, 1687-1745). */
typedef struct {
  void* ctx;
  int (*all_gather)(void* ctx, const void* send, void* recv, size_t bytes, void* cuda_stream);
  int (*barrier)(void* ctx, void* cuda_stream);
  int (*exchange)(void* ctx, const void* const* send_ptr, const size_t* send_bytes, void* const* recv_ptr,
                  const size_t* recv_bytes, void* cuda_stream);
} b2s_comm_ops;

/* Fills `ops` with the NCCL form of the table for one rank of `nccl_comm`.  `barrier_word` is one
 * zeroed int of device memory the barrier may use.  Release with b2s_nccl_comm_ops_release. */
int b2s_nccl_comm_ops(b2s_comm_ops* ops, void* nccl_comm, int rank, int nranks, void* barrier_word);
void b2s_nccl_comm_ops_release(b2s_comm_ops* ops);

/* A group of `nranks` ranks that are threads of the calling process, synchronised on the host:
 * fills ops_out[0..nranks-1], one table per rank, each to be used by one thread.  For hosts that
 * drive several streams or GPUs from one process, and for exercising the multi-rank paths on a
 * single GPU.  Every table is released with b2s_thread_comm_destroy. */
int b2s_thread_comm_create(int nranks, b2s_comm_ops* ops_out);
void b2s_thread_comm_destroy(b2s_comm_ops* ops);

/* Sorts a 1-D array whose contiguous tiles live on the `nranks` GPUs of one communicator: rank
 * r holds `n_local` elements starting at global position `global_offset`.  Every rank of the
 * communicator must call, even with n_local == 0 (src/cupynumeric/sort/sort_template.inl:62-72).
 * On return *out_ptr is a buffer from `alloc` holding *out_len elements - this rank's part of
 * the globally sorted values, or (argsort) of their int64 global indices; the parts of ranks
 * 0..nranks-1, concatenated, are the global stable sort.  The buffer belongs to the caller, as
 * with an unbound store's bind_data (sort.cu:1774-1783); *out_global_offset (may be NULL) is the
 * global position of its first element.  Synchronises the stream.
 *
 * How it works: samples of the unsorted tiles are gathered, weighted splitters are chosen from
 * them on the device, and each rank's partition kernel writes every element straight into the
 * receive buffer of its destination GPU (plain stores through a peer mapping of that buffer); after
 * one barrier each GPU sorts what it received.  The peer mappings need `alloc` to return cudaMalloc
 * memory that CUDA IPC can export (ranks in processes of their own) or ranks that share a process;
 * otherwise, when a receive buffer turns out too small, or with B2S_DIST_P2P=0 in the environment,
 * the partition is written locally and moved with the table's `exchange`.  The result is the same
 * either way.
 *
 * A failure that only one rank meets (its allocator returns NULL, a CUDA error) does not leave the
 * others waiting: the rank keeps taking part in the collectives, its status travels with the
 * gathered data and every rank returns the failure.
 * Replaces SortImplBody<GPU> for unbound 1-D outputs plus sample_sort_nccl_nd
 * (src/cupynumeric/sort/sort.cu:1797-1940 and 1270-1784). */
int b2s_dist_sort_1d_ops(int dtype, const void* keys_in, size_t n_local, int64_t global_offset, int argsort,
                         const b2s_comm_ops* ops, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                         void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void** out_ptr,
                         size_t* out_len, int64_t* out_global_offset, void* cuda_stream);
/* The same call with the NCCL form of the table built from `nccl_comm`. */
int b2s_dist_sort_1d(int dtype, const void* keys_in, size_t n_local, int64_t global_offset, int argsort,
                     void* nccl_comm, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                     void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void** out_ptr,
                     size_t* out_len, int64_t* out_global_offset, void* cuda_stream);

/* Moves the parts that b2s_dist_sort_1d left on the ranks (variable lengths, rank order) into
 * fixed extents: rank r ends up with the elements [out_global_start, out_global_start + out_len)
 * of the globally sorted sequence in `out`.  The extents of all ranks must tile the same range the
 * parts cover.  Every rank calls.  This is what a bound, aligned output store needs after a
 * sample sort along a split axis; it replaces rebalance_data
 * (src/cupynumeric/sort/sort.cu:799-1261) for one segment at a time.  Synchronises the stream. */
int b2s_dist_rebalance_1d_ops(size_t elem_bytes, const void* part, size_t part_len, int64_t part_global_start,
                              void* out, size_t out_len, int64_t out_global_start, const b2s_comm_ops* ops, int rank,
                              int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                              b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream);
int b2s_dist_rebalance_1d(size_t elem_bytes, const void* part, size_t part_len, int64_t part_global_start,
                          void* out, size_t out_len, int64_t out_global_start, void* nccl_comm, int rank,
                          int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                          b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream);

/* Sorts an N-D tile along its last axis when that axis is the one split over the ranks: every rank
 * holds the same `rows` rows and `extent_local` consecutive elements of each (slices in rank order,
 * dense row-major).  tile_out has the tile's shape and receives this rank's slice of every sorted
 * row - values, or (argsort) int64 positions along the whole axis.  All rows go through at once:
 * the rows are dealt out to the ranks, completed by one exchange, sorted by the segmented local
 * sort and returned by a second exchange; exact extents, no rebalancing step.  Every rank calls.
 * Worth it when there are at least as many rows as ranks; a few long rows are better served by
 * b2s_dist_sort_1d + b2s_dist_rebalance_1d per row.  Synchronises the stream.
 * Replaces sample_sort_nccl_nd + rebalance_data for this case
 * (src/cupynumeric/sort/sort.cu:1270-1784, 799-1261). */
int b2s_dist_sort_nd_ops(int dtype, const void* tile_in, void* tile_out, int argsort, size_t rows, size_t extent_local,
                         const b2s_comm_ops* ops, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                         void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream);
int b2s_dist_sort_nd(int dtype, const void* tile_in, void* tile_out, int argsort, size_t rows, size_t extent_local,
                     void* nccl_comm, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                     b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream);

/* Stable merge of `nruns` (<= 32) sorted runs, ties taken from the lower-numbered run first:
 * out receives the merged keys, or - when run_idx is not NULL - only the merged int64 payloads.
 * `ws`: b2s_kway_merge_workspace_bytes(total, nruns) bytes of device scratch.  One pass over the
 * data whatever the run count; stands where the reference has merge_all_buffers
 * (src/cupynumeric/sort/sort.cu:608-790).  b2s_local_sort uses it for 1-D tiles of 2^30 keys and
 * more (sorted in chunks); the distributed sort needs no merge. */
int b2s_kway_merge_workspace_bytes(size_t total, int nruns, size_t* bytes);
int b2s_kway_merge(int dtype, int nruns, const void* const* run_keys, const int64_t* const* run_idx,
                   const size_t* run_len, void* out, void* ws, size_t ws_bytes, void* cuda_stream);

/* NCCL communicator plumbing for hosts that are not Legate (which hands the task its
 * communicator: cupynumeric/_thunk/_sort.py:89-90, sort.cu:1923).  `id128` is the 128-byte
 * ncclUniqueId made on one rank and distributed by the caller. */
int b2s_nccl_unique_id(void* out128);
int b2s_nccl_comm_create(void** comm, int nranks, const void* id128, int rank);
int b2s_nccl_comm_destroy(void* comm);

/* Host-side pieces of the splitter logic, exported so that they can be exercised without a GPU.
 * A sample is the 48-byte record {uint64 okey_hi, okey_lo; int64 position; int64 weight; int32 rank;
 * int32 pad}: a key in its order-preserving unsigned form (okey_lo is used by 16-byte keys only),
 * its position in the owner's tile and the number of elements of that tile it stands for (0: slot
 * not populated).  Role of SegmentSample, src/cupynumeric/sort/sort.h:37-43. */
int b2s_samples_per_rank(void);
/* Position and weight of regular sample j of s in a tile of n >= s elements (the reference takes
 * its samples from the sorted tile, sort.cu:523-527; here they come from the unsorted one). */
long long b2s_host_sample_position(long long j, long long s, long long n);
long long b2s_host_sample_weight(long long j, long long s, long long n);
/* Orders `count` samples by (key, rank, position), unpopulated ones last
 * (SegmentSampleComparator, sort.h:60-81; thrust::stable_sort at sort.cu:1441-1445). */
void b2s_host_sort_samples(void* samples, size_t count);
/* Sorts the gathered samples and writes the nbuckets-1 splitters: splitter k is the first sample
 * at which the cumulative weight reaches k/nbuckets of the total (sort.cu:1455-1470 picks by
 * count; weights keep ragged tiles from skewing the cut). */
int b2s_host_select_splitters(void* samples, size_t count, int nbuckets, void* splitters_out);
/* Destination of the element (key, my_rank, pos): the number of splitters whose (key, rank,
 * position) triple is smaller than the element's (sort.h:72-78, sort.cu:170-187). */
int b2s_host_bucket_of(const void* splitters, int nsplit, int my_rank, unsigned long long okey_hi,
                       unsigned long long okey_lo, long long pos);

/* ---- SEARCHSORTED (the sorted output's natural consumer; a separate task in the reference) ---- */

/* For each of `num_values` values, combines this tile's contribution to its insertion position
 * in the global sorted array into `positions` (int64, one per value): left != 0 -> atomic MIN of
 * (lower bound + global_offset) when the lower bound lies inside the tile; left == 0 -> atomic
 * MAX of (upper bound + global_offset) when it is positive.  The caller pre-fills `positions`
 * with the global array size (left) or 0 (right) and reduces over ranks with MIN / MAX, exactly
 * the reduction stores of the reference task (src/cupynumeric/sort/searchsorted.cu:25-122,
 * cupynumeric/_thunk/deferred.py:5425-5451).  Keys compare in the sort's total order. */
int b2s_searchsorted(int dtype, const void* sorted_tile, size_t n_tile, int64_t global_offset,
                     const void* values, size_t num_values, int left, int64_t* positions,
                     void* cuda_stream);

/* ---- UNIQUE on sorted data ------------------------------------------------------------------- */

/* Writes the first element of every run of equal keys of `sorted` (n elements, ascending) to
 * `out` (room for n elements, must not alias `sorted`) and the number written to *out_len.
 * Keys are equal when the sort treats them as ties: one NaN, one zero.  After b2s_local_sort
 * this is the local half of the reference's UNIQUE task (thrust::sort + thrust::unique,
 * src/cupynumeric/set/unique.cu:150-208).  `ws`: b2s_unique_workspace_bytes(n) bytes, 256-byte
 * aligned.  Synchronises the stream (the count comes back to the host). */
int b2s_unique_workspace_bytes(size_t n, size_t* bytes);
int b2s_unique_sorted(int dtype, const void* sorted, size_t n, void* out, size_t* out_len, void* ws,
                      size_t ws_bytes, void* cuda_stream);

/* ---- PARTITION by selection, LEXSORT over several keys --------------------------------------- */

/* Partitions a 1-D tile around its element of rank `kth` (0-based, in the sort's total order)
 * without sorting it: keys_out (may be NULL) receives the elements below that key, then those equal
 * to it, then those above; idx_out (may be NULL) the positions (index_offset + i) in the same
 * arrangement.  The order inside the three blocks is unspecified, as numpy.partition allows.  A
 * radix select over the key bytes finds the key (one pass per byte), one more pass writes the
 * blocks.  keys_out must not be keys_in; n < 2^32.  `ws`: b2s_partition_workspace_bytes() bytes,
 * 256-byte aligned.  The reference sorts instead (cupynumeric/_thunk/deferred.py:5476-5494). */
int b2s_partition_workspace_bytes(size_t* bytes);
int b2s_partition_1d(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t n, size_t kth,
                     int64_t index_offset, void* ws, size_t ws_bytes, void* cuda_stream);

/* Indices that sort `nkeys` keys of the same shape lexicographically along the last axis, keys[0]
 * being the least significant (numpy.lexsort's convention): `volume` elements per key in
 * `volume / segment` rows; idx_out receives int64 positions inside each row.  One stable argsort per
 * key with the order so far carried through it; no step leaves the library.  `ws`:
 * b2s_lexsort_workspace_bytes(...) bytes, 256-byte aligned.  Replaces the chain of ARGSORT tasks
 * and gathers of cupynumeric/_module/ssc_sorting.py:423-444. */
int b2s_lexsort_workspace_bytes(int nkeys, const int* dtypes, size_t volume, size_t segment, size_t* bytes);
int b2s_lexsort(int nkeys, const int* dtypes, const void* const* keys, int64_t* idx_out, size_t volume, size_t segment,
                void* ws, size_t ws_bytes, void* cuda_stream);

/* ---- measurement aids (no counterpart in the reference, which relies on Legate's profiler,
 * cupynumeric/_utils/profiling.py:33-73) ------------------------------------------------------ */

/* Kernel families counted and timed separately. */
typedef enum {
  B2S_K_HIST    = 0, /* digit histograms */
  B2S_K_SCAN    = 1, /* histogram scan + pass routing */
  B2S_K_SWEEP   = 2, /* onesweep radix pass */
  B2S_K_FIXUP   = 3, /* leftover copies / synthesised indices */
  B2S_K_SEGSORT = 4, /* on-chip segmented sort */
  B2S_K_UNIT    = 5, /* segments of one element */
  B2S_K_DIST    = 6, /* sampling, splitter selection and counting kernels of the distributed sort */
  B2S_K_MERGE   = 7, /* k-way merge */
  B2S_K_XCHG    = 8, /* the partition kernel that writes into the destinations' receive buffers (or the collective exchange) */
  B2S_K_COUNT   = 9
} b2s_kernel_kind_t;

/* Switches per-launch CUDA-event timing on or off and forgets earlier records.  Process-wide,
 * not thread-safe: meant for a single-threaded benchmark harness. */
int b2s_profile_enable(int on);

/* Sum of the event-timed durations (ms) and number of launches of one kernel family since
 * b2s_profile_enable(1).  Waits for the recorded launches to finish. */
int b2s_profile_read(int kind, double* total_ms, unsigned long long* launches);

/* The same records one by one, in launch order: writes the durations (ms) of the first `capacity`
 * launches of the family to ms_out and the number of recorded launches to *launches (call with
 * capacity 0 to size the array).  A radix pass that the routing found it could skip still shows
 * up here, as a launch of a few microseconds. */
int b2s_profile_durations(int kind, float* ms_out, size_t capacity, size_t* launches);

/* Number of kernels of one family (or of all, kind < 0) this process has launched so far. */
unsigned long long b2s_launch_count(int kind);

#ifdef __cplusplus
}
#endif
#endif /* B200SORT_H_ */
