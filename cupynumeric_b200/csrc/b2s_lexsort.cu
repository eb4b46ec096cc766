// Lexicographic argsort over several keys along the last axis (the last key is the most
// significant): one stable radix argsort per key, least significant key first, each applied to
// that key gathered through the order found so far.  On 1-D tiles the 32-bit positions travel
// through the radix passes of every key as the payload, so a key costs one gather and one sort;
// nothing leaves the library between the keys (the reference chains argsort tasks and index
// gathers from Python, cupynumeric/_module/ssc_sorting.py:423-444).
#include <cuda_runtime.h>

#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_prof.h"

namespace b2s {
bool local_sort_pos32_supported(size_t n);
int local_sort_payload32(int dtype, const void* keys_in, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                         int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, int out32 = 0);

static size_t lex_elem_bytes(int dtype)
{
  switch (dtype) {
    case B2S_BOOL: case B2S_INT8: case B2S_UINT8: return 1;
    case B2S_INT16: case B2S_UINT16: case B2S_FLOAT16: return 2;
    case B2S_INT32: case B2S_UINT32: case B2S_FLOAT32: return 4;
    case B2S_INT64: case B2S_UINT64: case B2S_FLOAT64: case B2S_COMPLEX64: return 8;
    case B2S_COMPLEX128: return 16;
    default: return 0;
  }
}

// out[i] = in[row(i) * segment + order[i]]   (order holds positions inside the row)
template <typename T, typename I>
__global__ void lex_gather_kernel(const T* __restrict__ in, const I* __restrict__ order, size_t volume, size_t segment,
                                  T* __restrict__ out)
{
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < volume; i += stride)
    out[i] = in[(i / segment) * segment + (size_t)order[i]];
}

// order_out[i] = order_in[row(i) * segment + pick[i]]
__global__ void lex_compose_kernel(const int64_t* __restrict__ order_in, const int64_t* __restrict__ pick, size_t volume,
                                   size_t segment, int64_t* __restrict__ order_out)
{
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < volume; i += stride)
    order_out[i] = order_in[(i / segment) * segment + (size_t)pick[i]];
}

template <typename I>
static cudaError_t lex_gather(size_t eb, const void* in, const I* order, size_t volume, size_t segment, void* out,
                              cudaStream_t stream)
{
  prof::Scope ps(prof::K_FIXUP, stream);
  unsigned int grid = (unsigned int)((volume + 1023) / 1024);
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid == 0) grid = 1;
  switch (eb) {
    case 1: lex_gather_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(in), order, volume, segment, static_cast<uint8_t*>(out)); break;
    case 2: lex_gather_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(in), order, volume, segment, static_cast<uint16_t*>(out)); break;
    case 4: lex_gather_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(in), order, volume, segment, static_cast<uint32_t*>(out)); break;
    case 8: lex_gather_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint64_t*>(in), order, volume, segment, static_cast<uint64_t*>(out)); break;
    default: lex_gather_kernel<<<grid, 256, 0, stream>>>(static_cast<const ulonglong2*>(in), order, volume, segment, static_cast<ulonglong2*>(out)); break;
  }
  return cudaGetLastError();
}

struct LexLayout {
  size_t off_gather, off_ord[2], off_pick, off_sort, sort_bytes, total;
};

static int lex_layout(int nkeys, const int* dtypes, size_t volume, size_t segment, LexLayout* l)
{
  size_t max_eb = 0, max_ws = 0;
  for (int k = 0; k < nkeys; ++k) {
    const size_t eb = lex_elem_bytes(dtypes[k]);
    if (eb == 0) return B2S_ERR_UNSUPPORTED;
    size_t ws = 0;
    const int rc = b2s_workspace_bytes(dtypes[k], volume, segment, 1, &ws);
    if (rc != B2S_OK) return rc;
    max_eb = eb > max_eb ? eb : max_eb;
    max_ws = ws > max_ws ? ws : max_ws;
  }
  size_t off = 0;
  l->off_gather = off; off += align_up(volume * max_eb, 256);
  l->off_ord[0] = off; off += align_up(volume * 8, 256);
  l->off_ord[1] = off; off += align_up(volume * 8, 256);
  l->off_pick   = off; off += align_up(volume * 8, 256);
  l->off_sort   = off; off += align_up(max_ws, 256);
  l->sort_bytes = max_ws;
  l->total      = off;
  return B2S_OK;
}

}  // namespace b2s

using namespace b2s;

extern "C" {

int b2s_lexsort_workspace_bytes(int nkeys, const int* dtypes, size_t volume, size_t segment, size_t* bytes)
{
  if (nkeys < 1 || dtypes == nullptr || bytes == nullptr) return B2S_ERR_INVALID_ARG;
  if (volume > 0 && (segment == 0 || volume % segment != 0)) return B2S_ERR_INVALID_ARG;
  LexLayout l{};
  const int rc = lex_layout(nkeys, dtypes, volume, segment ? segment : 1, &l);
  if (rc == B2S_OK) *bytes = l.total;
  return rc;
}

int b2s_lexsort(int nkeys, const int* dtypes, const void* const* keys, int64_t* idx_out, size_t volume, size_t segment,
                void* ws, size_t ws_bytes, void* cuda_stream)
{
  if (nkeys < 1 || dtypes == nullptr || keys == nullptr) return B2S_ERR_INVALID_ARG;
  if (volume == 0) return B2S_OK;
  if (idx_out == nullptr || segment == 0 || volume % segment != 0) return B2S_ERR_INVALID_ARG;
  for (int k = 0; k < nkeys; ++k)
    if (keys[k] == nullptr) return B2S_ERR_INVALID_ARG;
  LexLayout l{};
  int rc = lex_layout(nkeys, dtypes, volume, segment, &l);
  if (rc != B2S_OK) return rc;
  if (ws == nullptr || ws_bytes < l.total || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  void* gathered      = base + l.off_gather;
  int64_t* ord[2]     = {reinterpret_cast<int64_t*>(base + l.off_ord[0]), reinterpret_cast<int64_t*>(base + l.off_ord[1])};
  int64_t* pick       = reinterpret_cast<int64_t*>(base + l.off_pick);
  void* sort_ws       = base + l.off_sort;
  const int one_d     = volume == segment;

  // 1-D tiles of a size the single radix sort takes (and no 16-byte keys): the order so far rides
  // through the passes as a 32-bit payload
  bool carry = one_d && local_sort_pos32_supported(volume);
  for (int k = 0; k < nkeys; ++k) carry = carry && dtypes[k] != B2S_COMPLEX128;
  if (carry) {
    uint32_t* pos[2] = {reinterpret_cast<uint32_t*>(ord[0]), reinterpret_cast<uint32_t*>(ord[1])};
    int cur = 0;
    for (int k = 0; k < nkeys; ++k) {
      const bool last = k == nkeys - 1;
      const void* src = keys[k];
      if (k > 0) {
        if (lex_gather<uint32_t>(lex_elem_bytes(dtypes[k]), keys[k], pos[cur], volume, segment, gathered, stream) != cudaSuccess)
          return B2S_ERR_CUDA;
        src = gathered;
      }
      if (last) {
        rc = local_sort_payload32(dtypes[k], src, k == 0 ? nullptr : pos[cur], idx_out, volume, 0, sort_ws, l.sort_bytes, stream);
      } else {
        rc = local_sort_payload32(dtypes[k], src, k == 0 ? nullptr : pos[cur], reinterpret_cast<int64_t*>(pos[cur ^ 1]), volume, 0,
                                  sort_ws, l.sort_bytes, stream, 1);
        cur ^= 1;
      }
      if (rc != B2S_OK) return rc;
    }
    return B2S_OK;
  }

  // every other shape: argsort of the gathered key, then the order so far taken through it
  int cur = 0;
  for (int k = 0; k < nkeys; ++k) {
    const bool last = k == nkeys - 1;
    if (k == 0) {
      rc = b2s_local_sort(dtypes[0], keys[0], nullptr, last ? idx_out : ord[cur], volume, segment, 0, one_d, 1, sort_ws, l.sort_bytes, stream);
      if (rc != B2S_OK) return rc;
      continue;
    }
    if (lex_gather<int64_t>(lex_elem_bytes(dtypes[k]), keys[k], ord[cur], volume, segment, gathered, stream) != cudaSuccess) return B2S_ERR_CUDA;
    rc = b2s_local_sort(dtypes[k], gathered, nullptr, pick, volume, segment, 0, one_d, 1, sort_ws, l.sort_bytes, stream);
    if (rc != B2S_OK) return rc;
    {
      prof::Scope ps(prof::K_FIXUP, stream);
      unsigned int grid = (unsigned int)((volume + 1023) / 1024);
      if (grid > 148 * 16) grid = 148 * 16;
      lex_compose_kernel<<<grid, 256, 0, stream>>>(ord[cur], pick, volume, segment, last ? idx_out : ord[cur ^ 1]);
      if (cudaGetLastError() != cudaSuccess) return B2S_ERR_CUDA;
    }
    cur ^= 1;
  }
  return B2S_OK;
}
}
