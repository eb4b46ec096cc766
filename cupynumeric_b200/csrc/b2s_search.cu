// SEARCHSORTED: for every value, its insertion position in a sorted 1-D array that may be tiled
// over ranks.  Same per-tile contract as the reference's kernels
// (src/cupynumeric/sort/searchsorted.cu:25-74): a tile contributes its lower bound (left) only
// when it lies inside the tile, its upper bound (right) only when it is positive, shifted by
// the tile's global offset, and contributions combine by MIN (left) / MAX (right) into an
// output the caller pre-filled with the global size (left) or 0 (right).  Keys compare in the
// same total order the sort produces (NaN last).
#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_prof.h"

namespace b2s {

template <int KB>
__global__ void __launch_bounds__(256)
searchsorted_kernel(const typename KeyOf<KB>::type* __restrict__ sorted, long long n, long long global_offset,
                    const typename KeyOf<KB>::type* __restrict__ values, long long num_values, int left, int xf,
                    long long* __restrict__ positions)
{
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_values) return;
  const auto v = to_ordered_rt<KB>(values[i], xf);
  long long lo = 0, hi = n;
  while (lo < hi) {
    const long long mid = lo + ((hi - lo) >> 1);
    const auto k        = to_ordered_rt<KB>(sorted[mid], xf);
    const bool go_right = left ? (k < v) : (k <= v);
    if (go_right) lo = mid + 1; else hi = mid;
  }
  if (left) {
    if (lo < n) atomicMin(positions + i, lo + global_offset);
  } else {
    if (lo > 0) atomicMax(positions + i, lo + global_offset);
  }
}

}  // namespace b2s

using namespace b2s;

extern "C" int b2s_searchsorted(int dtype, const void* sorted_tile, size_t n_tile, int64_t global_offset,
                                const void* values, size_t num_values, int left, int64_t* positions,
                                void* cuda_stream)
{
  int kb = 0, xf = 0;
  switch (dtype) {
    case B2S_BOOL: case B2S_UINT8: kb = 1; xf = XF_UNSIGNED; break;
    case B2S_INT8: kb = 1; xf = XF_SIGNED; break;
    case B2S_UINT16: kb = 2; xf = XF_UNSIGNED; break;
    case B2S_INT16: kb = 2; xf = XF_SIGNED; break;
    case B2S_FLOAT16: kb = 2; xf = XF_FLOAT; break;
    case B2S_UINT32: kb = 4; xf = XF_UNSIGNED; break;
    case B2S_INT32: kb = 4; xf = XF_SIGNED; break;
    case B2S_FLOAT32: kb = 4; xf = XF_FLOAT; break;
    case B2S_UINT64: kb = 8; xf = XF_UNSIGNED; break;
    case B2S_INT64: kb = 8; xf = XF_SIGNED; break;
    case B2S_FLOAT64: kb = 8; xf = XF_FLOAT; break;
    case B2S_COMPLEX64: kb = 8; xf = XF_CFLOAT; break;
    default: return B2S_ERR_UNSUPPORTED;
  }
  if (num_values == 0) return B2S_OK;
  if (values == nullptr || positions == nullptr || (n_tile > 0 && sorted_tile == nullptr)) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  const unsigned int grid = (unsigned int)((num_values + 255) / 256);
  long long* pos = reinterpret_cast<long long*>(positions);
  prof::Scope ps(prof::K_DIST, stream);
  switch (kb) {
    case 1: searchsorted_kernel<1><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(sorted_tile), (long long)n_tile, global_offset, static_cast<const uint8_t*>(values), (long long)num_values, left, xf, pos); break;
    case 2: searchsorted_kernel<2><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(sorted_tile), (long long)n_tile, global_offset, static_cast<const uint16_t*>(values), (long long)num_values, left, xf, pos); break;
    case 4: searchsorted_kernel<4><<<grid, 256, 0, stream>>>(static_cast<const uint32_t*>(sorted_tile), (long long)n_tile, global_offset, static_cast<const uint32_t*>(values), (long long)num_values, left, xf, pos); break;
    default: searchsorted_kernel<8><<<grid, 256, 0, stream>>>(static_cast<const uint64_t*>(sorted_tile), (long long)n_tile, global_offset, static_cast<const uint64_t*>(values), (long long)num_values, left, xf, pos); break;
  }
  return cudaGetLastError() == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}
