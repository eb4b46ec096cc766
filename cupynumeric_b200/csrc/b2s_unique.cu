// UNIQUE on sorted data: keeps the first element of every run of equal keys.  With the sort in
// front of it this replaces the local part of the reference's UNIQUE task, which is a
// thrust::sort followed by thrust::unique (src/cupynumeric/set/unique.cu:150-208).  Keys are
// equal when their ordered images are equal: all NaNs are one value, -0.0 equals +0.0.
#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_prof.h"

namespace b2s {

constexpr int UQ_THREADS = 256;
constexpr int UQ_ITEMS   = 16;
constexpr int UQ_TILE    = UQ_THREADS * UQ_ITEMS;

template <int KB>
__device__ __forceinline__ bool is_head(const typename KeyOf<KB>::type* a, long long i, int xf)
{
  return i == 0 || to_ordered_rt<KB>(a[i], xf) != to_ordered_rt<KB>(a[i - 1], xf);
}

// pass 1: heads per tile
template <int KB>
__global__ void __launch_bounds__(UQ_THREADS)
unique_count_kernel(const typename KeyOf<KB>::type* __restrict__ a, long long n, int xf,
                    unsigned int* __restrict__ tile_counts)
{
  const long long base = (long long)blockIdx.x * UQ_TILE;
  unsigned int c       = 0;
  for (int j = 0; j < UQ_ITEMS; ++j) {
    const long long i = base + j * UQ_THREADS + threadIdx.x;
    if (i < n && is_head<KB>(a, i, xf)) ++c;
  }
  c = __reduce_add_sync(0xFFFFFFFFu, c);
  __shared__ unsigned int w[UQ_THREADS / 32];
  if ((threadIdx.x & 31) == 0) w[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int t = 0;
    for (int k = 0; k < UQ_THREADS / 32; ++k) t += w[k];
    tile_counts[blockIdx.x] = t;
  }
}

// pass 2 (one CTA): exclusive scan of the tile counts into 64-bit offsets; total at [ntiles]
static __global__ void __launch_bounds__(1024)
unique_scan_kernel(const unsigned int* __restrict__ tile_counts, long long ntiles, unsigned long long* __restrict__ offsets)
{
  __shared__ unsigned long long warp_tot[32];
  __shared__ unsigned long long carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (long long base = 0; base < ntiles; base += 1024) {
    const long long i      = base + threadIdx.x;
    const unsigned long long c = i < ntiles ? tile_counts[i] : 0;
    unsigned long long incl    = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[w] = incl;
    __syncthreads();
    unsigned long long before = carry;
    for (int k = 0; k < w; ++k) before += warp_tot[k];
    if (i < ntiles) offsets[i] = before + incl - c;
    __syncthreads();
    if (threadIdx.x == 1023) carry = before + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) offsets[ntiles] = carry;
}

// pass 3: write the heads of a tile to its offset, in order
template <int KB>
__global__ void __launch_bounds__(UQ_THREADS)
unique_write_kernel(const typename KeyOf<KB>::type* __restrict__ a, long long n, int xf,
                    const unsigned long long* __restrict__ offsets, typename KeyOf<KB>::type* __restrict__ out)
{
  using K = typename KeyOf<KB>::type;
  __shared__ unsigned int warp_tot[UQ_THREADS / 32];
  __shared__ unsigned int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const long long base           = (long long)blockIdx.x * UQ_TILE;
  const unsigned long long tile0 = offsets[blockIdx.x];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int j = 0; j < UQ_ITEMS; ++j) {
    const long long i = base + j * UQ_THREADS + threadIdx.x;
    const bool head   = i < n && is_head<KB>(a, i, xf);
    const unsigned int bal = __ballot_sync(0xFFFFFFFFu, head);
    if (lane == 0) warp_tot[w] = __popc(bal);
    __syncthreads();
    unsigned int before = running;
    for (int k = 0; k < w; ++k) before += warp_tot[k];
    if (head) out[tile0 + before + __popc(bal & ((1u << lane) - 1))] = a[i];
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int t = 0;
      for (int k = 0; k < UQ_THREADS / 32; ++k) t += warp_tot[k];
      running += t;
    }
    __syncthreads();
  }
}

template <int KB>
static cudaError_t unique_launch(const void* a, long long n, int xf, void* out, unsigned char* ws, cudaStream_t stream)
{
  using K = typename KeyOf<KB>::type;
  const long long ntiles        = (n + UQ_TILE - 1) / UQ_TILE;
  unsigned int* counts          = reinterpret_cast<unsigned int*>(ws);
  unsigned long long* offsets   = reinterpret_cast<unsigned long long*>(ws + align_up((size_t)ntiles * 4, 256));
  {
    prof::Scope ps(prof::K_DIST, stream);
    unique_count_kernel<KB><<<(unsigned int)ntiles, UQ_THREADS, 0, stream>>>(static_cast<const K*>(a), n, xf, counts);
  }
  {
    prof::Scope ps(prof::K_DIST, stream);
    unique_scan_kernel<<<1, 1024, 0, stream>>>(counts, ntiles, offsets);
  }
  {
    prof::Scope ps(prof::K_DIST, stream);
    unique_write_kernel<KB><<<(unsigned int)ntiles, UQ_THREADS, 0, stream>>>(static_cast<const K*>(a), n, xf, offsets,
                                                                          static_cast<K*>(out));
  }
  return cudaGetLastError();
}

}  // namespace b2s

using namespace b2s;

extern "C" {

int b2s_unique_workspace_bytes(size_t n, size_t* bytes)
{
  if (bytes == nullptr) return B2S_ERR_INVALID_ARG;
  const size_t ntiles = (n + UQ_TILE - 1) / UQ_TILE;
  *bytes              = align_up(ntiles * 4, 256) + align_up((ntiles + 1) * 8, 256);
  return B2S_OK;
}

int b2s_unique_sorted(int dtype, const void* sorted, size_t n, void* out, size_t* out_len, void* ws,
                      size_t ws_bytes, void* cuda_stream)
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
  if (out_len == nullptr) return B2S_ERR_INVALID_ARG;
  *out_len = 0;
  if (n == 0) return B2S_OK;
  size_t need = 0;
  b2s_unique_workspace_bytes(n, &need);
  if (sorted == nullptr || out == nullptr || out == sorted) return B2S_ERR_INVALID_ARG;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u)) return B2S_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  unsigned char* w    = static_cast<unsigned char*>(ws);
  cudaError_t e;
  switch (kb) {
    case 1: e = unique_launch<1>(sorted, (long long)n, xf, out, w, stream); break;
    case 2: e = unique_launch<2>(sorted, (long long)n, xf, out, w, stream); break;
    case 4: e = unique_launch<4>(sorted, (long long)n, xf, out, w, stream); break;
    default: e = unique_launch<8>(sorted, (long long)n, xf, out, w, stream); break;
  }
  if (e != cudaSuccess) return B2S_ERR_CUDA;
  const size_t ntiles = (n + UQ_TILE - 1) / UQ_TILE;
  unsigned long long total = 0;
  const unsigned long long* offsets = reinterpret_cast<const unsigned long long*>(w + align_up(ntiles * 4, 256));
  if (cudaMemcpyAsync(&total, offsets + ntiles, 8, cudaMemcpyDeviceToHost, stream) != cudaSuccess) return B2S_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return B2S_ERR_CUDA;
  *out_len = (size_t)total;
  return B2S_OK;
}
}
