// complex128 keys (complex64 is an 8-byte radix key of its own, XF_CFLOAT, and does not come
// here): lexicographic (real, imaginary) order, the order the reference's Thrust path
// uses for complex64/128 (src/cupynumeric/sort/thrust_sort.cuh:61-123 with the comparison of
// src/cupynumeric/binary/binary_op_util.h:32-36).  Done as two stable radix argsorts - by the
// imaginary parts, then by the real parts in that order - which is the lexicographic order.  On
// 1-D tiles the order found by the first sort rides through the passes of the second one as a
// 32-bit payload (no 64-bit indices in any pass, no composition of two permutations).
#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_prof.h"

namespace b2s {
bool local_sort_pos32_supported(size_t n);
int local_sort_payload32(int dtype, const void* keys_in, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                         int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, int out32 = 0);

template <typename F>
__global__ void cplx_split_kernel(const F* __restrict__ c, F* __restrict__ re, F* __restrict__ im, size_t n)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    re[i] = c[2 * i];
    im[i] = c[2 * i + 1];
  }
}

// out[i] = src[segment start of i + idx[i]]
template <typename F>
__global__ void cplx_gather_kernel(const F* __restrict__ src, const int64_t* __restrict__ idx, F* __restrict__ out,
                                   size_t n, size_t seg)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = src[i / seg * seg + (size_t)idx[i]];
}

// 1-D, 32-bit positions: out[i] = src[pos[i]]
template <typename F>
__global__ void cplx_gather32_kernel(const F* __restrict__ src, const uint32_t* __restrict__ pos, F* __restrict__ out, size_t n)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = src[pos[i]];
}

// 1-D, 32-bit positions of the final order: the indices and/or the sorted complex values.  The
// values come from the interleaved input, one 16-byte access per element when VEC (input and
// output 16-byte aligned), which touches half the sectors of two 8-byte gathers.
template <typename F, bool VEC>
__global__ void cplx_finish32_kernel(const F* __restrict__ c_in, const uint32_t* __restrict__ pos, F* __restrict__ c_out,
                                     int64_t* __restrict__ idx_out, size_t n, int64_t index_offset)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t j = pos[i];
    if (idx_out) idx_out[i] = (int64_t)j + index_offset;
    if (c_out) {
      if (VEC) {
        reinterpret_cast<double2*>(c_out)[i] = __ldg(reinterpret_cast<const double2*>(c_in) + j);
      } else {
        c_out[2 * i]     = c_in[2 * j];
        c_out[2 * i + 1] = c_in[2 * j + 1];
      }
    }
  }
}

// the same from the split copies (the sort is in place: the interleaved input is being overwritten)
template <typename F>
__global__ void cplx_finish_split32_kernel(const F* __restrict__ re, const F* __restrict__ im, const uint32_t* __restrict__ pos,
                                           F* __restrict__ c_out, int64_t* __restrict__ idx_out, size_t n, int64_t index_offset)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t j = pos[i];
    if (idx_out) idx_out[i] = (int64_t)j + index_offset;
    if (c_out) {
      c_out[2 * i]     = re[j];
      c_out[2 * i + 1] = im[j];
    }
  }
}

// Composes the two permutations and writes the indices and/or the sorted complex values.
template <typename F>
__global__ void cplx_finish_kernel(const F* __restrict__ re, const F* __restrict__ im,
                                   const int64_t* __restrict__ idx1, const int64_t* __restrict__ idx2,
                                   F* __restrict__ c_out, int64_t* __restrict__ idx_out, size_t n, size_t seg,
                                   int64_t index_offset)
{
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t s0 = i / seg * seg;
    const size_t j  = (size_t)idx1[s0 + (size_t)idx2[i]];
    if (idx_out) idx_out[i] = (int64_t)j + index_offset;
    if (c_out) {
      c_out[2 * i]     = re[s0 + j];
      c_out[2 * i + 1] = im[s0 + j];
    }
  }
}

struct CplxLayout {
  size_t inner, off_re, off_im, off_re1, off_idx1, off_idx2, total;
};

static int cplx_layout(int dtype, size_t volume, size_t segment, CplxLayout* l)
{
  const int part  = dtype == B2S_COMPLEX64 ? B2S_FLOAT32 : B2S_FLOAT64;
  const size_t fb = dtype == B2S_COMPLEX64 ? 4 : 8;
  int rc          = b2s_workspace_bytes(part, volume, segment, 1, &l->inner);
  if (rc != B2S_OK) return rc;
  size_t off = align_up(l->inner, 256);
  l->off_re  = off; off += align_up(volume * fb, 256);
  l->off_im  = off; off += align_up(volume * fb, 256);
  l->off_re1 = off; off += align_up(volume * fb, 256);
  l->off_idx1 = off; off += align_up(volume * 8, 256);
  l->off_idx2 = off; off += align_up(volume * 8, 256);
  l->total = off;
  return B2S_OK;
}

int complex_ws_bytes(int dtype, size_t volume, size_t segment, size_t* bytes)
{
  CplxLayout l{};
  int rc = cplx_layout(dtype, volume, segment, &l);
  if (rc == B2S_OK) *bytes = l.total;
  return rc;
}

template <typename F>
static int complex_sort_t(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                          size_t segment, int64_t index_offset, unsigned char* ws, cudaStream_t stream)
{
  CplxLayout l{};
  int rc = cplx_layout(dtype, volume, segment, &l);
  if (rc != B2S_OK) return rc;
  const int part = dtype == B2S_COMPLEX64 ? B2S_FLOAT32 : B2S_FLOAT64;
  F* re          = reinterpret_cast<F*>(ws + l.off_re);
  F* im          = reinterpret_cast<F*>(ws + l.off_im);
  F* re1         = reinterpret_cast<F*>(ws + l.off_re1);
  int64_t* idx1  = reinterpret_cast<int64_t*>(ws + l.off_idx1);
  int64_t* idx2  = reinterpret_cast<int64_t*>(ws + l.off_idx2);
  const int one_d = volume == segment;
  unsigned int grid = (unsigned int)((volume + 1023) / 1024);
  if (grid > 148 * 16) grid = 148 * 16;
  {
    prof::Scope ps(prof::K_FIXUP, stream);
    cplx_split_kernel<F><<<grid, 256, 0, stream>>>(static_cast<const F*>(keys_in), re, im, volume);
  }
  if (one_d && local_sort_pos32_supported(volume)) {
    uint32_t* pos1 = reinterpret_cast<uint32_t*>(idx1);
    uint32_t* pos2 = reinterpret_cast<uint32_t*>(idx2);
    rc = local_sort_payload32(part, im, nullptr, reinterpret_cast<int64_t*>(pos1), volume, 0, ws, l.inner, stream, 1);
    if (rc != B2S_OK) return rc;
    {
      prof::Scope ps(prof::K_FIXUP, stream);
      cplx_gather32_kernel<F><<<grid, 256, 0, stream>>>(re, pos1, re1, volume);
    }
    rc = local_sort_payload32(part, re1, pos1, reinterpret_cast<int64_t*>(pos2), volume, 0, ws, l.inner, stream, 1);
    if (rc != B2S_OK) return rc;
    {
      prof::Scope ps(prof::K_FIXUP, stream);
      // in place (keys_out == keys_in) the values are taken from the split copies instead
      const bool vec = sizeof(F) == 8 && keys_out != keys_in && ((reinterpret_cast<uintptr_t>(keys_in) | reinterpret_cast<uintptr_t>(keys_out)) & 15u) == 0;
      if (keys_out == keys_in)
        cplx_finish_split32_kernel<F><<<grid, 256, 0, stream>>>(re, im, pos2, static_cast<F*>(keys_out), idx_out, volume, index_offset);
      else if (vec)
        cplx_finish32_kernel<F, true><<<grid, 256, 0, stream>>>(static_cast<const F*>(keys_in), pos2, static_cast<F*>(keys_out), idx_out, volume, index_offset);
      else
        cplx_finish32_kernel<F, false><<<grid, 256, 0, stream>>>(static_cast<const F*>(keys_in), pos2, static_cast<F*>(keys_out), idx_out, volume, index_offset);
    }
    return cudaGetLastError() == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
  }
  rc = b2s_local_sort(part, im, nullptr, idx1, volume, segment, 0, one_d, 1, ws, l.inner, stream);
  if (rc != B2S_OK) return rc;
  {
    prof::Scope ps(prof::K_FIXUP, stream);
    cplx_gather_kernel<F><<<grid, 256, 0, stream>>>(re, idx1, re1, volume, segment);
  }
  rc = b2s_local_sort(part, re1, nullptr, idx2, volume, segment, 0, one_d, 1, ws, l.inner, stream);
  if (rc != B2S_OK) return rc;
  {
    prof::Scope ps(prof::K_FIXUP, stream);
    cplx_finish_kernel<F><<<grid, 256, 0, stream>>>(re, im, idx1, idx2, static_cast<F*>(keys_out), idx_out, volume,
                                                    segment, index_offset);
  }
  return cudaGetLastError() == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

int complex_local_sort(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                       size_t segment, int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream)
{
  if (volume == 0) return B2S_OK;
  if (keys_in == nullptr || (keys_out == nullptr && idx_out == nullptr)) return B2S_ERR_INVALID_ARG;
  if (segment == 0 || volume % segment != 0) return B2S_ERR_INVALID_ARG;
  size_t need = 0;
  int rc      = complex_ws_bytes(dtype, volume, segment, &need);
  if (rc != B2S_OK) return rc;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  if (dtype == B2S_COMPLEX64)
    return complex_sort_t<float>(dtype, keys_in, keys_out, idx_out, volume, segment, index_offset,
                                 static_cast<unsigned char*>(ws), stream);
  return complex_sort_t<double>(dtype, keys_in, keys_out, idx_out, volume, segment, index_offset,
                                static_cast<unsigned char*>(ws), stream);
}

}  // namespace b2s
