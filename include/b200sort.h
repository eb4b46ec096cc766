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
 *     patterns preserved.
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
  B2S_K_DIST    = 6, /* sampling, splitter search and cut kernels of the distributed sort */
  B2S_K_MERGE   = 7, /* k-way merge */
  B2S_K_COUNT   = 8
} b2s_kernel_kind_t;

/* Switches per-launch CUDA-event timing on or off and forgets earlier records.  Process-wide,
 * not thread-safe: meant for a single-threaded benchmark harness. */
int b2s_profile_enable(int on);

/* Sum of the event-timed durations (ms) and number of launches of one kernel family since
 * b2s_profile_enable(1).  Waits for the recorded launches to finish. */
int b2s_profile_read(int kind, double* total_ms, unsigned long long* launches);

/* Number of kernels of one family (or of all, kind < 0) this process has launched so far. */
unsigned long long b2s_launch_count(int kind);

#ifdef __cplusplus
}
#endif
#endif /* B200SORT_H_ */
