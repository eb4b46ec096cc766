// A variant of the 1-D / segmented local sort for callers that must not allocate device memory.
//
// Some hosts of this library have no allocator to offer at the moment they need a sort: a task
// body running under a runtime that forbids cudaMalloc/cudaFree while tasks are in flight (both
// calls synchronise the whole device and bypass the runtime's memory accounting), a thread
// whose pool is exhausted or not yet created, or a library that is itself called from such a
// place.  For them the scratch memory of the radix sort lives here, in a fixed device array that
// every GPU loading this library carries from load to exit.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/b200sort.h"

namespace {

// Scratch of the sort kernels: control block, look-back table and the ping-pong copies of keys
// and indices.  B2S_NOALLOC_SCRATCH_BYTES (32 MiB) is enough for, e.g., 2^20 eight-byte keys
// with indices, or 2^21 four-byte keys without.
static __device__ __align__(256) unsigned char g_scratch[B2S_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
// Device address of g_scratch per device, filled on the first call made on that device.  In
// host code `g_scratch` itself is only a handle for the runtime, not an address a kernel may use.
unsigned char* g_scratch_addr[MAX_DEVICES] = {};
std::mutex g_setup_mutex;  // two host threads may make their first call on a device together

// One-time set-up per device, with that device current: looks the array's device address up.
int scratch_of_current_device(unsigned char** out)
{
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return B2S_ERR_CUDA;
  if (dev < 0 || dev >= MAX_DEVICES) return B2S_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_scratch) != cudaSuccess || p == nullptr) return B2S_ERR_CUDA;
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return B2S_OK;
}

}  // namespace

extern "C" int b2s_local_sort_noalloc(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out,
                                      size_t volume, size_t segment, int64_t index_offset, int ndim_is_1,
                                      void* cuda_stream)
{
  size_t need = 0;
  int rc      = b2s_workspace_bytes(dtype, volume, segment, idx_out != nullptr, &need);
  if (rc != B2S_OK) return rc;
  if (need > (size_t)B2S_NOALLOC_SCRATCH_BYTES) return B2S_ERR_WORKSPACE;  // problem too large for the fixed scratch
  unsigned char* scratch = nullptr;
  rc = scratch_of_current_device(&scratch);
  if (rc != B2S_OK) return rc;
  // b2s_local_sort clears the control block and the look-back table of the scratch on every call
  return b2s_local_sort(dtype, keys_in, keys_out, idx_out, volume, segment, index_offset, ndim_is_1, 1, scratch,
                        (size_t)B2S_NOALLOC_SCRATCH_BYTES, cuda_stream);
}

// The status word of the last b2s_local_sort_noalloc on this device sits at the head of the same
// array; this reads it back the way b2s_check_status does for a caller-owned workspace.
extern "C" int b2s_noalloc_check_status(void* cuda_stream)
{
  unsigned char* scratch = nullptr;
  const int rc = scratch_of_current_device(&scratch);
  if (rc != B2S_OK) return rc;
  return b2s_check_status(scratch, cuda_stream);
}
