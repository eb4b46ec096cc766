// extern "C" entry points of the local sort (declared in include/b200sort.h).
#include "../../include/b200sort.h"
#include <cstdlib>

#include "b2s_launch.cuh"

namespace b2s {

struct DtypeInfo {
  int kb;
  int xf;
};

// Key width and ordering rule per element type; complex128 is not a radix key (16 bytes).
inline bool dtype_info(int dtype, DtypeInfo* o)
{
  switch (dtype) {
    case B2S_BOOL: *o = {1, XF_UNSIGNED}; return true;
    case B2S_INT8: *o = {1, XF_SIGNED}; return true;
    case B2S_INT16: *o = {2, XF_SIGNED}; return true;
    case B2S_INT32: *o = {4, XF_SIGNED}; return true;
    case B2S_INT64: *o = {8, XF_SIGNED}; return true;
    case B2S_UINT8: *o = {1, XF_UNSIGNED}; return true;
    case B2S_UINT16: *o = {2, XF_UNSIGNED}; return true;
    case B2S_UINT32: *o = {4, XF_UNSIGNED}; return true;
    case B2S_UINT64: *o = {8, XF_UNSIGNED}; return true;
    case B2S_FLOAT16: *o = {2, XF_FLOAT}; return true;
    case B2S_FLOAT32: *o = {4, XF_FLOAT}; return true;
    case B2S_FLOAT64: *o = {8, XF_FLOAT}; return true;
    case B2S_COMPLEX64: *o = {8, XF_CFLOAT}; return true;  // (real, imaginary) as one 8-byte key
    default: return false;
  }
}

inline size_t radix_ws(int kb, size_t n, bool pairs)
{
  switch (kb) {
    case 1: return radix_1d_layout<1>(n, pairs).total;
    case 2: return radix_1d_layout<2>(n, pairs).total;
    case 4: return radix_1d_layout<4>(n, pairs).total;
    default: return radix_1d_layout<8>(n, pairs).total;
  }
}

inline cudaError_t radix_any(int kb, int xf, const void* in, void* out, int64_t* idx, unsigned int n,
                             int64_t off, unsigned char* ws, cudaStream_t s, int idx32 = 0,
                             const uint32_t* idx_in = nullptr, const unsigned int* hp = nullptr, int hn = 0)
{
  switch (kb) {
    case 1: return launch_radix_1d<1>(xf, in, out, idx, n, off, ws, s, idx32, idx_in, hp, hn);
    case 2: return launch_radix_1d<2>(xf, in, out, idx, n, off, ws, s, idx32, idx_in, hp, hn);
    case 4: return launch_radix_1d<4>(xf, in, out, idx, n, off, ws, s, idx32, idx_in, hp, hn);
    default: return launch_radix_1d<8>(xf, in, out, idx, n, off, ws, s, idx32, idx_in, hp, hn);
  }
}

inline size_t radix_seg_ws(int kb, size_t seg_len, size_t nseg, bool pairs)
{
  switch (kb) {
    case 1: return radix_seg_layout<1>(seg_len, nseg, pairs).total;
    case 2: return radix_seg_layout<2>(seg_len, nseg, pairs).total;
    case 4: return radix_seg_layout<4>(seg_len, nseg, pairs).total;
    default: return radix_seg_layout<8>(seg_len, nseg, pairs).total;
  }
}

inline cudaError_t radix_seg_any(int kb, int xf, const void* in, void* out, int64_t* idx, unsigned int seg_len,
                                 unsigned int nseg, int64_t off, unsigned char* ws, cudaStream_t s)
{
  switch (kb) {
    case 1: return launch_radix_seg<1>(xf, in, out, idx, seg_len, nseg, off, ws, s);
    case 2: return launch_radix_seg<2>(xf, in, out, idx, seg_len, nseg, off, ws, s);
    case 4: return launch_radix_seg<4>(xf, in, out, idx, seg_len, nseg, off, ws, s);
    default: return launch_radix_seg<8>(xf, in, out, idx, seg_len, nseg, off, ws, s);
  }
}

inline cudaError_t seg_any(int kb, int xf, const void* in, void* out, int64_t* idx, unsigned int L,
                           unsigned long long nseg, int64_t off, Ctrl* ctrl, cudaStream_t s)
{
  switch (kb) {
    case 1: return launch_segsort<1>(xf, in, out, idx, L, nseg, off, ctrl, s);
    case 2: return launch_segsort<2>(xf, in, out, idx, L, nseg, off, ctrl, s);
    case 4: return launch_segsort<4>(xf, in, out, idx, L, nseg, off, ctrl, s);
    default: return launch_segsort<8>(xf, in, out, idx, L, nseg, off, ctrl, s);
  }
}

// Segments of one element: the output is the input, every index is index_offset.
__global__ void unit_segment_kernel(const unsigned char* in, unsigned char* out, int64_t* idx, size_t volume,
                                    int kb, int64_t index_offset)
{
  const size_t gthread = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gstride = (size_t)gridDim.x * blockDim.x;
  if (out != nullptr && out != in)
    for (size_t i = gthread; i < volume * kb; i += gstride) out[i] = in[i];
  if (idx != nullptr)
    for (size_t i = gthread; i < volume; i += gstride) idx[i] = index_offset;
}

// Several segments longer than the on-chip kernel takes go through the segmented onesweep; its
// element offsets are 32-bit, so one call takes fewer than 2^32 elements.
constexpr size_t MAX_SEG_VOLUME = (size_t)1 << 32;

}  // namespace b2s

namespace b2s {
int complex_ws_bytes(int dtype, size_t volume, size_t segment, size_t* bytes);
int complex_local_sort(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                       size_t segment, int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream);
// ---- 1-D arrays at or above the single-sort limit: sort chunks, then merge them ----
// The look-back counts of the radix passes are 30-bit, so one radix sort takes fewer than 2^30
// keys.  Longer 1-D tiles are cut into chunks of half that, each chunk is sorted on its own and
// the sorted chunks (at most 32) go through the stable k-way merge in chunk order, which keeps
// the whole sort stable.  B2S_MAX_1D_LOG2 lowers the limit (a testing aid).
inline size_t single_sort_limit()
{
  const char* e = std::getenv("B2S_MAX_1D_LOG2");
  if (e != nullptr) {
    const int v = std::atoi(e);
    if (v >= 10 && v <= 30) return (size_t)1 << v;
  }
  return MAX_N_1D;
}

struct ChunkLayout {
  size_t chunk, nchunks, inner, off_keys, off_idx, off_cuts, cuts_bytes, total;
};

inline int chunk_layout(int dtype, int kb, size_t n, bool argsort, ChunkLayout* l)
{
  l->chunk   = single_sort_limit() / 2;
  l->nchunks = (n + l->chunk - 1) / l->chunk;
  if (l->nchunks > 32) return B2S_ERR_UNSUPPORTED;
  l->inner = radix_ws(kb, l->chunk, argsort);
  (void)dtype;
  size_t off  = align_up(l->inner, 256);
  l->off_keys = off; off += align_up(n * kb, 256);
  l->off_idx  = off; if (argsort) off += align_up(n * 8, 256);
  b2s_kway_merge_workspace_bytes(n, (int)l->nchunks, &l->cuts_bytes);
  l->off_cuts = off; off += align_up(l->cuts_bytes, 256);
  l->total = off;
  return B2S_OK;
}


// Sizes the single radix sort takes with 32-bit payloads carried through its passes.
bool local_sort_pos32_supported(size_t n) { return n > SEG_CAP && n < single_sort_limit(); }

// Stable 1-D argsort of keys that carry a 32-bit payload each (pay_in[i] belongs to keys_in[i];
// null: the payload of element i is i).  out32 == 0: idx_out[k] = index_offset + payload of the
// k-th smallest key, as int64; out32 != 0: idx_out points to n uint32 values that receive the bare
// payloads.  The distributed sort uses it on what a rank received (payload = global position minus a
// common base), the lexicographic sort to carry its order from key to key: travelling as 32 bits the
// payload costs the radix passes no more than a plain argsort.
int local_sort_payload32(int dtype, const void* keys_in, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                         int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, int out32)
{
  DtypeInfo di;
  if (!dtype_info(dtype, &di) || !local_sort_pos32_supported(n)) return B2S_ERR_UNSUPPORTED;
  if (keys_in == nullptr || idx_out == nullptr) return B2S_ERR_INVALID_ARG;
  size_t need = 0;
  int rc      = b2s_workspace_bytes(dtype, n, n, 1, &need);
  if (rc != B2S_OK) return rc;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  const cudaError_t e = radix_any(di.kb, di.xf, keys_in, nullptr, idx_out, (unsigned int)n, index_offset,
                                  static_cast<unsigned char*>(ws), stream, out32 ? 1 : 0, pay_in);
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

// Stable 1-D sort of what a rank of the distributed sort received: keys only (keys_out) or an
// argsort with the 32-bit payloads carried through the passes (pay_in, idx_out).  The digit
// histograms of the keys come ready-made in `nparts` pieces, counted by the senders.
int local_sort_received(int dtype, const void* keys_in, void* keys_out, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                        int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, const unsigned int* hist_parts,
                        int nparts)
{
  DtypeInfo di;
  if (!dtype_info(dtype, &di) || !local_sort_pos32_supported(n)) return B2S_ERR_UNSUPPORTED;
  if (keys_in == nullptr || (keys_out == nullptr) == (idx_out == nullptr)) return B2S_ERR_INVALID_ARG;
  size_t need = 0;
  int rc      = b2s_workspace_bytes(dtype, n, n, idx_out != nullptr, &need);
  if (rc != B2S_OK) return rc;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  const cudaError_t e = radix_any(di.kb, di.xf, keys_in, keys_out, idx_out, (unsigned int)n, index_offset,
                                  static_cast<unsigned char*>(ws), stream, 0, pay_in, hist_parts, nparts);
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

}  // namespace b2s

using namespace b2s;

extern "C" {

const char* b2s_status_string(int status)
{
  switch (status) {
    case B2S_OK: return "ok";
    case B2S_ERR_INVALID_ARG: return "invalid argument";
    case B2S_ERR_CUDA: return "CUDA error";
    case B2S_ERR_NCCL: return "NCCL error";
    case B2S_ERR_WORKSPACE: return "workspace too small or misaligned";
    case B2S_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case B2S_ERR_UNSUPPORTED: return "unsupported dtype or shape";
    default: return "unknown status";
  }
}

int b2s_version(void) { return 100; }

int b2s_workspace_bytes(int dtype, size_t volume, size_t segment, int argsort, size_t* bytes)
{
  DtypeInfo di;
  if (bytes == nullptr) return B2S_ERR_INVALID_ARG;
  if (dtype == B2S_COMPLEX128) {
    if (volume > 0 && (segment == 0 || volume % segment != 0)) return B2S_ERR_INVALID_ARG;
    return complex_ws_bytes(dtype, volume, segment, bytes);
  }
  if (!dtype_info(dtype, &di)) return B2S_ERR_UNSUPPORTED;
  if (volume > 0 && (segment == 0 || volume % segment != 0)) return B2S_ERR_INVALID_ARG;
  size_t need = align_up(sizeof(Ctrl), 256);
  if (volume > 0 && segment > SEG_CAP) {
    if (volume == segment && segment >= single_sort_limit()) {
      ChunkLayout cl{};
      const int rc = chunk_layout(dtype, di.kb, segment, argsort != 0, &cl);
      if (rc != B2S_OK) return rc;
      need = cl.total;
    } else if (segment >= MAX_N_1D) {
      return B2S_ERR_UNSUPPORTED;
    } else if (volume == segment) {
      need = radix_ws(di.kb, segment, argsort != 0);
    } else {
      if (volume >= MAX_SEG_VOLUME) return B2S_ERR_UNSUPPORTED;
      need = radix_seg_ws(di.kb, segment, volume / segment, argsort != 0);
    }
  }
  *bytes = need;
  return B2S_OK;
}

int b2s_local_sort(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t volume,
                   size_t segment, int64_t index_offset, int ndim_is_1, int stable, void* ws, size_t ws_bytes,
                   void* cuda_stream)
{
  (void)stable;  // always stable
  DtypeInfo di;
  if (dtype == B2S_COMPLEX128) {
    if (ndim_is_1 && volume != segment) return B2S_ERR_INVALID_ARG;
    return complex_local_sort(dtype, keys_in, keys_out, idx_out, volume, segment, index_offset, ws, ws_bytes,
                              static_cast<cudaStream_t>(cuda_stream));
  }
  if (!dtype_info(dtype, &di)) return B2S_ERR_UNSUPPORTED;
  if (volume == 0) return B2S_OK;
  if (keys_in == nullptr || (keys_out == nullptr && idx_out == nullptr)) return B2S_ERR_INVALID_ARG;
  if (segment == 0 || volume % segment != 0) return B2S_ERR_INVALID_ARG;
  const size_t nseg = volume / segment;
  if (ndim_is_1 && nseg != 1) return B2S_ERR_INVALID_ARG;
  size_t need = 0;
  int rc      = b2s_workspace_bytes(dtype, volume, segment, idx_out != nullptr, &need);
  if (rc != B2S_OK) return rc;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  Ctrl* ctrl          = static_cast<Ctrl*>(ws);
  cudaError_t e;

  if (segment <= SEG_CAP) {
    e = cudaMemsetAsync(ctrl, 0, sizeof(Ctrl), stream);
    if (e != cudaSuccess) return B2S_ERR_CUDA;
    if (segment == 1) {
      size_t grid = (volume + 4095) / 4096;
      if (grid > 148 * 8) grid = 148 * 8;
      prof::Scope ps(prof::K_UNIT, stream);
      unit_segment_kernel<<<(unsigned int)grid, 256, 0, stream>>>(static_cast<const unsigned char*>(keys_in),
                                                                 static_cast<unsigned char*>(keys_out), idx_out,
                                                                 volume, di.kb, index_offset);
      return cudaGetLastError() == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
    }
    e = seg_any(di.kb, di.xf, keys_in, keys_out, idx_out, (unsigned int)segment, nseg, index_offset, ctrl, stream);
    return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
  }

  if (nseg == 1 && segment >= single_sort_limit()) {
    ChunkLayout cl{};
    rc = chunk_layout(dtype, di.kb, segment, idx_out != nullptr, &cl);
    if (rc != B2S_OK) return rc;
    unsigned char* base = static_cast<unsigned char*>(ws);
    unsigned char* sk   = base + cl.off_keys;
    int64_t* si         = idx_out ? reinterpret_cast<int64_t*>(base + cl.off_idx) : nullptr;
    const void* run_keys[32];
    const int64_t* run_idx[32];
    size_t run_len[32];
    for (size_t c = 0; c < cl.nchunks; ++c) {
      const size_t lo = c * cl.chunk, len = (lo + cl.chunk <= segment) ? cl.chunk : segment - lo;
      e = radix_any(di.kb, di.xf, static_cast<const unsigned char*>(keys_in) + lo * di.kb, sk + lo * di.kb,
                    si ? si + lo : nullptr, (unsigned int)len, index_offset + (int64_t)lo, base, stream);
      if (e != cudaSuccess) return B2S_ERR_CUDA;
      run_keys[c] = sk + lo * di.kb;
      run_idx[c]  = si ? si + lo : nullptr;
      run_len[c]  = len;
    }
    if (idx_out != nullptr) {
      rc = b2s_kway_merge(dtype, (int)cl.nchunks, run_keys, run_idx, run_len, idx_out, base + cl.off_cuts, cl.cuts_bytes,
                          cuda_stream);
      if (rc != B2S_OK) return rc;
    }
    if (keys_out != nullptr) {
      rc = b2s_kway_merge(dtype, (int)cl.nchunks, run_keys, nullptr, run_len, keys_out, base + cl.off_cuts, cl.cuts_bytes,
                          cuda_stream);
      if (rc != B2S_OK) return rc;
    }
    return B2S_OK;
  } else if (nseg == 1) {
    e = radix_any(di.kb, di.xf, keys_in, keys_out, idx_out, (unsigned int)segment, index_offset,
                  static_cast<unsigned char*>(ws), stream);
  } else {
    e = radix_seg_any(di.kb, di.xf, keys_in, keys_out, idx_out, (unsigned int)segment, (unsigned int)nseg,
                      index_offset, static_cast<unsigned char*>(ws), stream);
  }
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

// Self-test of the bounded waits.  Sorts a small array of its own whose first tile is never
// processed (the tile tickets of the first pass start at 1), with a poll limit of a few thousand:
// every later tile waits for the first tile's look-back entry, gives up within milliseconds,
// records DEV_ERR_TIMEOUT and raises the abort flag; the remaining passes see the flag and
// return.  Nothing traps, faults or waits without a bound; the workspace and the context stay usable.
namespace b2s {
__global__ void selftest_fill_kernel(uint32_t* keys, unsigned int n)
{
  for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) keys[i] = i * 2654435761u;
}
}  // namespace b2s

int b2s_selftest_wait_timeout(void* ws, size_t ws_bytes, void* cuda_stream)
{
  constexpr unsigned int N = 1u << 16;  // a dozen tiles
  const auto lay           = radix_1d_layout<4>(N, false);
  const size_t need        = lay.total + 2 * (size_t)N * 4;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  Ctrl* ctrl          = reinterpret_cast<Ctrl*>(base);
  uint32_t* in        = reinterpret_cast<uint32_t*>(base + lay.total);
  uint32_t* out       = in + N;
  unsigned int* lb    = reinterpret_cast<unsigned int*>(base + lay.off_lookback);
  if (cudaMemsetAsync(base, 0, lay.off_keys[0], stream) != cudaSuccess) return B2S_ERR_CUDA;
  selftest_fill_kernel<<<64, 256, 0, stream>>>(in, N);
  RouteArgs ra{};
  ra.keys_in     = in;
  ra.keys_out    = out;
  ra.tmp_keys[0] = base + lay.off_keys[0];
  ra.tmp_keys[1] = base + lay.off_keys[1];
  ra.n           = N;
  ra.npass       = 4;
  ra.key_bytes   = 4;
  hist_kernel<4, XF_UNSIGNED><<<16, HIST_THREADS, 0, stream>>>(in, N, ctrl, ra);
  // the sabotage: the first pass hands out tickets 1, 2, ... so that tile 0 is never taken, and a
  // short poll limit
  const unsigned int one = 1, limit = 4096;
  if (cudaMemcpyAsync(&ctrl->tile_counter[0], &one, 4, cudaMemcpyHostToDevice, stream) != cudaSuccess) return B2S_ERR_CUDA;
  if (cudaMemcpyAsync(&ctrl->spin_limit, &limit, 4, cudaMemcpyHostToDevice, stream) != cudaSuccess) return B2S_ERR_CUDA;
  const SegGeom geo{N, lay.tiles, 1u, 4, nullptr};
  const cudaError_t e = launch_sweeps<4, XF_UNSIGNED, false>(ctrl, lb, lay.tiles, geo, 0, stream);
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

int b2s_check_status(void* ws, void* cuda_stream)
{
  if (ws == nullptr) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  unsigned int st     = 0;
  if (cudaMemcpyAsync(&st, &static_cast<Ctrl*>(ws)->status, sizeof(st), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
    return B2S_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return B2S_ERR_CUDA;
  return (int)st;
}
}
