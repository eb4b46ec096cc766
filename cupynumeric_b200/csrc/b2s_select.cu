// Selection instead of sorting for partition / argpartition of a 1-D tile: a most-significant-digit
// radix select finds the key of rank kth (one histogram launch per key byte; each descends only
// into the digit that holds the rank), then one pass writes the elements below that key, equal to
// it and above it as three blocks.  O(n) bytes instead of a full sort.  The reference sorts
// ("fallback to sort for now", cupynumeric/_thunk/deferred.py:5476-5494).
#include <cuda_runtime.h>

#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_prof.h"

namespace b2s {

struct SelectState {
  unsigned long long prefix;     // the digits of the rank-kth key found so far (ordered image, high digits)
  unsigned long long rank;       // rank still to resolve among the keys that match the prefix
  unsigned long long below;      // keys known to be smaller than every key that matches the prefix
  unsigned int hist[RADIX];      // digit counts of the pass in flight
  unsigned int done;             // CTAs of the pass in flight that have added their counts
  unsigned int equal;            // after the last pass: keys equal to the rank-kth key
  unsigned int cursor[3];        // write cursors of the three output blocks
  unsigned int pad_;
};

constexpr int SEL_THREADS = 512;

static int sel_kb_of(int dtype, int* xf)
{
  switch (dtype) {
    case B2S_BOOL: *xf = XF_UNSIGNED; return 1;
    case B2S_INT8: *xf = XF_SIGNED; return 1;
    case B2S_UINT8: *xf = XF_UNSIGNED; return 1;
    case B2S_INT16: *xf = XF_SIGNED; return 2;
    case B2S_UINT16: *xf = XF_UNSIGNED; return 2;
    case B2S_FLOAT16: *xf = XF_FLOAT; return 2;
    case B2S_INT32: *xf = XF_SIGNED; return 4;
    case B2S_UINT32: *xf = XF_UNSIGNED; return 4;
    case B2S_FLOAT32: *xf = XF_FLOAT; return 4;
    case B2S_INT64: *xf = XF_SIGNED; return 8;
    case B2S_UINT64: *xf = XF_UNSIGNED; return 8;
    case B2S_FLOAT64: *xf = XF_FLOAT; return 8;
    case B2S_COMPLEX64: *xf = XF_CFLOAT; return 8;
    default: return 0;
  }
}

// Pass `pass` (0 = most significant byte): counts the digit of every key whose higher digits equal
// the prefix; the CTA that finishes last picks the digit that holds the rank.
template <int KB>
__global__ void __launch_bounds__(SEL_THREADS)
select_pass_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned long long n, int xf, int pass, SelectState* st)
{
  using K = typename KeyOf<KB>::type;
  __shared__ unsigned int sh[RADIX];
  __shared__ int is_last;
  const int tid = threadIdx.x;
  if (tid < RADIX) sh[tid] = 0;
  __syncthreads();
  const int shift                 = 8 * (KB - 1 - pass);
  const unsigned long long prefix = st->prefix;
  // bits above the digit of this pass
  const unsigned long long himask = pass == 0 ? 0ull : (~0ull << (shift + 8)) & (KB == 8 ? ~0ull : ((1ull << (8 * KB)) - 1));
  auto look = [&](K raw) {
    const unsigned long long o = (unsigned long long)to_ordered_rt<KB>(raw, xf);
    if ((o & himask) == prefix) atomicAdd(&sh[(unsigned int)(o >> shift) & 0xFFu], 1u);
  };
  // 16-byte loads, four in flight per thread: after the first pass almost no key matches the prefix
  // and the pass is a plain read of the input
  constexpr int VEC    = 16 / KB;
  constexpr int UNROLL = 4;
  const bool aligned   = (reinterpret_cast<uintptr_t>(keys) & 15u) == 0;
  const unsigned long long nvec    = aligned ? n / VEC : 0;
  const unsigned long long gthread = (unsigned long long)blockIdx.x * SEL_THREADS + tid;
  const unsigned long long stride  = (unsigned long long)gridDim.x * SEL_THREADS;
  const uint4* vkeys               = reinterpret_cast<const uint4*>(keys);
  unsigned long long v             = gthread;
  for (; v + (UNROLL - 1) * stride < nvec; v += UNROLL * stride) {
    uint4 q[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) q[u] = __ldg(vkeys + v + u * stride);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      alignas(16) K tmp[VEC];
      *reinterpret_cast<uint4*>(tmp) = q[u];
#pragma unroll
      for (int j = 0; j < VEC; ++j) look(tmp[j]);
    }
  }
  for (; v < nvec; v += stride) {
    alignas(16) K tmp[VEC];
    *reinterpret_cast<uint4*>(tmp) = __ldg(vkeys + v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) look(tmp[j]);
  }
  for (unsigned long long i = nvec * VEC + gthread; i < n; i += stride) look(keys[i]);
  __syncthreads();
  if (tid < RADIX && sh[tid]) atomicAdd(&st->hist[tid], sh[tid]);
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(&st->done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // one warp walks the 256 counts: the digit whose cumulative count first exceeds the rank
  if (tid < 32) {
    unsigned int c[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      c[j] = st->hist[tid * 8 + j];
      sum += c[j];
    }
    unsigned int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (tid >= o) incl += t;
    }
    unsigned long long run       = incl - sum;  // keys in lower digit groups
    const unsigned long long rank = st->rank;
    int found = -1;
    unsigned long long before = 0;
    unsigned int count = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (found < 0 && rank >= run && rank < run + c[j]) {
        found  = tid * 8 + j;
        before = run;
        count  = c[j];
      }
      run += c[j];
    }
    if (found >= 0) {  // exactly one lane
      st->prefix = prefix | ((unsigned long long)found << shift);
      st->rank   = rank - before;
      st->below += before;
      st->equal  = count;
    }
  }
  __syncthreads();
  if (tid < RADIX) st->hist[tid] = 0;
  if (tid == 0) st->done = 0;
}

// Three blocks: [keys below the pivot][keys equal to it][keys above it]; the order inside a block is
// whatever the CTAs' reservations make it (a partition promises no more).  Every thread counts its
// elements per block in one packed word (three 16-bit fields), one scan of those words over the CTA
// gives every element its place in the CTA's three pieces, the pieces are put together in shared
// memory and written out as three runs of consecutive elements.
constexpr int P3_ITEMS = 8;
constexpr int P3_TILE  = SEL_THREADS * P3_ITEMS;

template <int KB>
__global__ void __launch_bounds__(SEL_THREADS, 3)
partition3_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned long long n, int xf, SelectState* st,
                  typename KeyOf<KB>::type* __restrict__ out_keys, int64_t* __restrict__ out_idx, int64_t index_offset)
{
  using K  = typename KeyOf<KB>::type;
  using OK = typename KeyOf<(KB <= 4 ? 4 : 8)>::type;  // comparisons of short keys stay 32-bit
  constexpr int WARPS = SEL_THREADS / 32;
  constexpr unsigned int F1 = 1u << 10, F2 = 1u << 20;  // a warp holds at most 256 elements: 10-bit fields
  __shared__ K skey[P3_TILE];
  __shared__ unsigned short ssrc[P3_TILE];     // where in the tile the staged element came from
  __shared__ unsigned int wtot[WARPS];
  __shared__ unsigned int base[3];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const OK pivot                 = (OK)st->prefix;
  const unsigned long long tile0 = (unsigned long long)blockIdx.x * P3_TILE;
  const unsigned int valid       = (unsigned int)min((unsigned long long)P3_TILE, n - tile0);
  const K* src                   = keys + tile0;
  K key[P3_ITEMS];
  unsigned int incs[P3_ITEMS];  // 0: no element; else the element's class as its counter increment
  unsigned int cnt = 0;
#pragma unroll
  for (int i = 0; i < P3_ITEMS; ++i) {
    const unsigned int e = i * SEL_THREADS + tid;
    incs[i]              = 0;
    if (e < valid) {
      key[i]     = src[e];
      const OK o = (OK)to_ordered_rt<KB>(key[i], xf);
      incs[i]    = o < pivot ? 1u : (o == pivot ? F1 : F2);
      cnt += incs[i];
    }
  }
  // exclusive prefix of the packed counts: inside the warp on the packed word, over the warps on
  // the three unpacked totals
  unsigned int incl = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) wtot[warp] = incl;
  __syncthreads();
  unsigned int b0 = 0, b1 = 0, b2 = 0, t0 = 0, t1 = 0, t2 = 0;  // elements of lower warps / of the CTA, per class
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    const unsigned int t = wtot[w];
    const unsigned int c0 = t & 0x3FFu, c1 = (t >> 10) & 0x3FFu, c2 = t >> 20;
    if (w < warp) {
      b0 += c0;
      b1 += c1;
      b2 += c2;
    }
    t0 += c0;
    t1 += c1;
    t2 += c2;
  }
  // the reservation travels to L2 and back while the tile is being staged
  unsigned int reserved = 0;
  if (tid < 3) {
    const unsigned int mine = tid == 0 ? t0 : (tid == 1 ? t1 : t2);
    if (mine) reserved = atomicAdd(&st->cursor[tid], mine);
  }
  // my first place in each of the CTA's three pieces (pieces start at 0, t0, t0 + t1)
  const unsigned int excl = incl - cnt;
  unsigned int p0 = b0 + (excl & 0x3FFu), p1 = t0 + b1 + ((excl >> 10) & 0x3FFu), p2 = t0 + t1 + b2 + (excl >> 20);
  const bool want_idx = out_idx != nullptr;
#pragma unroll
  for (int i = 0; i < P3_ITEMS; ++i) {
    if (incs[i]) {
      unsigned int p;
      if (incs[i] == 1u) p = p0++; else if (incs[i] == F1) p = p1++; else p = p2++;
      skey[p] = key[i];
      if (want_idx) ssrc[p] = (unsigned short)(i * SEL_THREADS + tid);
    }
  }
  if (tid < 3) base[tid] = reserved;
  __syncthreads();
  // the staged tile goes out as three runs of consecutive elements
  const unsigned long long below = st->below, equal = st->equal;
  const unsigned long long d0 = base[0], d1 = below + base[1] - t0, d2 = below + equal + base[2] - (t0 + t1);
  for (unsigned int p = tid; p < valid; p += SEL_THREADS) {
    const unsigned long long at = (p < t0 ? d0 : (p < t0 + t1 ? d1 : d2)) + p;
    if (out_keys != nullptr) out_keys[at] = skey[p];
    if (want_idx) out_idx[at] = index_offset + (int64_t)(tile0 + ssrc[p]);
  }
}

template <int KB>
static cudaError_t run_partition(const void* keys_in, void* keys_out, int64_t* idx_out, size_t n, size_t kth, int xf,
                                 int64_t index_offset, SelectState* st, cudaStream_t stream)
{
  using K = typename KeyOf<KB>::type;
  SelectState init{};
  init.rank = kth;
  cudaError_t e = cudaMemcpyAsync(st, &init, sizeof(init), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  unsigned int grid = (unsigned int)((n + SEL_THREADS * 16 - 1) / (SEL_THREADS * 16));
  if (grid > (unsigned int)sms * 4) grid = sms * 4;
  for (int pass = 0; pass < KB; ++pass) {
    prof::Scope ps(prof::K_HIST, stream);
    select_pass_kernel<KB><<<grid, SEL_THREADS, 0, stream>>>(static_cast<const K*>(keys_in), n, xf, pass, st);
  }
  {
    prof::Scope ps(prof::K_FIXUP, stream);
    const unsigned int tiles = (unsigned int)((n + P3_TILE - 1) / P3_TILE);
    partition3_kernel<KB><<<tiles, SEL_THREADS, 0, stream>>>(static_cast<const K*>(keys_in), n, xf, st, static_cast<K*>(keys_out),
                                                             idx_out, index_offset);
  }
  return cudaGetLastError();
}

}  // namespace b2s

using namespace b2s;

extern "C" {

int b2s_partition_workspace_bytes(size_t* bytes)
{
  if (bytes == nullptr) return B2S_ERR_INVALID_ARG;
  *bytes = align_up(sizeof(SelectState), 256);
  return B2S_OK;
}

int b2s_partition_1d(int dtype, const void* keys_in, void* keys_out, int64_t* idx_out, size_t n, size_t kth,
                     int64_t index_offset, void* ws, size_t ws_bytes, void* cuda_stream)
{
  int xf       = 0;
  const int kb = sel_kb_of(dtype, &xf);
  if (kb == 0) return B2S_ERR_UNSUPPORTED;
  if (n == 0) return B2S_OK;
  if (keys_in == nullptr || (keys_out == nullptr && idx_out == nullptr) || kth >= n) return B2S_ERR_INVALID_ARG;
  if (keys_out == keys_in) return B2S_ERR_INVALID_ARG;  // the input is read again while the output is written
  if (n >= ((size_t)1 << 32)) return B2S_ERR_UNSUPPORTED;
  if (ws == nullptr || ws_bytes < sizeof(SelectState) || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return B2S_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  SelectState* st     = static_cast<SelectState*>(ws);
  cudaError_t e;
  switch (kb) {
    case 1: e = run_partition<1>(keys_in, keys_out, idx_out, n, kth, xf, index_offset, st, stream); break;
    case 2: e = run_partition<2>(keys_in, keys_out, idx_out, n, kth, xf, index_offset, st, stream); break;
    case 4: e = run_partition<4>(keys_in, keys_out, idx_out, n, kth, xf, index_offset, st, stream); break;
    default: e = run_partition<8>(keys_in, keys_out, idx_out, n, kth, xf, index_offset, st, stream); break;
  }
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}
}
