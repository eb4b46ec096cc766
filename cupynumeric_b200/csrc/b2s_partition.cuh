// Partition kernels of the distributed sort for up to 8 destinations and keys of at most 8 bytes
// (the 8 GPUs of one NVSwitch box): every thread owns 16 CONSECUTIVE elements of the tile and
// counts its elements per destination in registers (eight 16-bit fields in two 64-bit words), so
// the stable rank of an element needs no warp vote and no shared-memory counter: it is the
// thread's exclusive prefix (one scan of the packed words over the CTA) plus a running count.
// Wider groups and 16-byte keys take the vote-based kernels beside the callers of these.
#pragma once
#include "b2s_common.cuh"
#include "b2s_dist_host.h"

namespace b2s {

constexpr int FP_THREADS = 256;
constexpr int FP_ITEMS   = 16;
constexpr int FP_TILE    = FP_THREADS * FP_ITEMS;
constexpr int FP_WARPS   = FP_THREADS / 32;
constexpr int FP_NB      = 8;  // destinations (padded)
constexpr unsigned long long FP_ONES = 0x0001000100010001ull;

// ordered key as narrow as the key itself: comparisons of 4-byte keys stay 32-bit
template <int KB> struct FpKey {
  using Raw = typename KeyOf<KB>::type;
  using OK  = typename KeyOf<(KB <= 4 ? 4 : 8)>::type;
  static __device__ __forceinline__ OK okey(Raw r, int xf) { return (OK)to_ordered_rt<KB>(r, xf); }
};

// The splitters of one tile in shared memory: ordered key and the tile-relative position that
// breaks ties (-1: every equal key lies right of the splitter; INT_MAX: none does).  Only the tile
// that holds a splitter's own element has a tie position inside it; for every other tile "right of
// the splitter" is a comparison of keys alone, k > adj with adj = key - 1 where the equal keys lie
// right.  `simple` says that all seven comparisons of this tile can be made that way.
template <int KB> struct FpSplit {
  typename FpKey<KB>::OK okey[FP_NB];
  typename FpKey<KB>::OK adj[FP_NB];
  int tie[FP_NB];
  int simple;
};

// Called by all threads of the CTA; the caller's __syncthreads() comes after it.  `simple` is
// cleared by the last __syncthreads() user of the previous tile at the earliest, set here by
// thread FP_NB and lowered by threads 0..FP_NB-1 after a barrier of their warp.
template <int KB>
__device__ __forceinline__ void fp_load_splitters(FpSplit<KB>* s, const LocalSplitter* __restrict__ split, long long tile_base,
                                                  int tid)
{
  using OK = typename FpKey<KB>::OK;
  if (tid < 32) {
    OK k  = (OK)~(OK)0;
    int t = 0x7FFFFFFF;
    if (tid < FP_NB - 1) {
      const LocalSplitter l = split[tid];
      if (l.valid) {
        k                  = (OK)l.okey.hi;
        const long long rel = l.tie_pos - tile_base;
        t                  = rel < 0 ? -1 : (rel > 0x7FFFFFFFll ? 0x7FFFFFFF : (int)rel);
      }
    }
    // equal keys all right (t < 0, needs key - 1 to exist) or all left (t beyond the tile)
    const bool plain = t < 0 ? k != (OK)0 : t >= FP_TILE - 1;
    const bool all   = __all_sync(0xFFFFFFFFu, tid >= FP_NB || plain);
    if (tid < FP_NB) {
      s->okey[tid] = k;
      s->adj[tid]  = t < 0 ? (OK)(k - (OK)1) : k;
      s->tie[tid]  = t;
    }
    if (tid == 0) s->simple = all ? 1 : 0;
  }
}

// number of splitters the element lies right of: three branch-free steps over the seven
// (padded) splitters.  An invalid splitter holds the largest key and INT_MAX: nothing is right of it.
template <int KB>
__device__ __forceinline__ unsigned int fp_classify(const FpSplit<KB>* s, typename FpKey<KB>::OK k, int pos_in_tile)
{
  unsigned int b = 0;
#pragma unroll
  for (int step = 2; step >= 0; --step) {
    const unsigned int mid = b + (1u << step) - 1u;
    const auto sk          = s->okey[mid];
    const int st           = s->tie[mid];
    const bool right       = k > sk || (k == sk && pos_in_tile > st);
    b += right ? (1u << step) : 0u;
  }
  return b;
}

// the same for a tile whose FpSplit is `simple`: keys alone decide
template <int KB>
__device__ __forceinline__ unsigned int fp_classify_simple(const FpSplit<KB>* s, typename FpKey<KB>::OK k)
{
  unsigned int b = 0;
#pragma unroll
  for (int step = 2; step >= 0; --step) b += k > s->adj[b + (1u << step) - 1u] ? (1u << step) : 0u;
  return b;
}

// 16 consecutive keys of a thread: 16-byte loads when `vec` (full tile, 16-byte aligned source; the
// source may be shared memory, so these are plain loads), guarded element loads otherwise
template <int KB>
__device__ __forceinline__ void fp_load_keys(typename FpKey<KB>::Raw (&key)[FP_ITEMS], const typename FpKey<KB>::Raw* src,
                                             int first, int valid, bool vec)
{
  using Raw = typename FpKey<KB>::Raw;
  if (vec) {
    constexpr int NV = FP_ITEMS * KB / 16;
    const uint4* v   = reinterpret_cast<const uint4*>(src + first);
    union {
      uint4 q[NV];
      Raw r[FP_ITEMS];
    } u;
#pragma unroll
    for (int j = 0; j < NV; ++j) u.q[j] = v[j];
#pragma unroll
    for (int i = 0; i < FP_ITEMS; ++i) key[i] = u.r[i];
  } else {
#pragma unroll
    for (int i = 0; i < FP_ITEMS; ++i) key[i] = first + i < valid ? src[first + i] : (Raw)0;
  }
}

__device__ __forceinline__ void fp_count(unsigned long long& lo, unsigned long long& hi, unsigned int b, bool live)
{
  const unsigned long long inc = live ? 1ull << ((b & 3u) * 16u) : 0ull;
  lo += b < 4u ? inc : 0ull;
  hi += b < 4u ? 0ull : inc;
}
__device__ __forceinline__ unsigned int fp_field(unsigned long long lo, unsigned long long hi, unsigned int b)
{
  return (unsigned int)((b < 4u ? lo : hi) >> ((b & 3u) * 16u)) & 0xFFFFu;
}

// Tiles are grouped into chunks for the scan over tiles: the counting kernel adds every tile's
// counts to its chunk's sums, the scan kernel starts every chunk from the sums of the chunks before it.
constexpr int FP_CHUNK_TILES = 256;

// per-tile element counts per destination: tile_counts[tile * FP_NB + b].  Counting does not care
// which thread looks at which element, so the loads are striped over the CTA: consecutive threads
// load consecutive 16-byte vectors.
template <int KB>
__global__ void __launch_bounds__(FP_THREADS)
part_count_fast_kernel(const typename FpKey<KB>::Raw* __restrict__ keys, long long n, int xf,
                       const LocalSplitter* __restrict__ split, unsigned int* __restrict__ tile_counts,
                       unsigned long long* __restrict__ chunk_sums)
{
  using Raw = typename FpKey<KB>::Raw;
  __shared__ FpSplit<KB> ss;
  __shared__ unsigned int cnt[FP_NB];
  const int tid        = threadIdx.x;
  const long long base = (long long)blockIdx.x * FP_TILE;
  fp_load_splitters<KB>(&ss, split, base, tid);
  if (tid < FP_NB) cnt[tid] = 0;
  __syncthreads();
  const int valid = (int)min((long long)FP_TILE, n - base);
  const bool vec  = valid == FP_TILE && ((reinterpret_cast<uintptr_t>(keys + base) & 15u) == 0);
  constexpr int VEC = 16 / KB;               // keys per 16-byte vector
  constexpr int NV  = FP_ITEMS / VEC;        // vectors per thread
  unsigned long long lo = 0, hi = 0;
  if (vec) {
    union {
      uint4 q;
      Raw r[VEC];
    } u[NV];
    const uint4* v = reinterpret_cast<const uint4*>(keys + base);
#pragma unroll
    for (int j = 0; j < NV; ++j) u[j].q = __ldg(v + j * FP_THREADS + tid);
    if (ss.simple) {  // the same for the whole CTA
#pragma unroll
      for (int j = 0; j < NV; ++j) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) fp_count(lo, hi, fp_classify_simple<KB>(&ss, FpKey<KB>::okey(u[j].r[k], xf)), true);
      }
    } else {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const int e = (j * FP_THREADS + tid) * VEC + k;
          fp_count(lo, hi, fp_classify<KB>(&ss, FpKey<KB>::okey(u[j].r[k], xf), e), true);
        }
      }
    }
  } else {
#pragma unroll 4
    for (int i = 0; i < FP_ITEMS; ++i) {
      const int e = i * FP_THREADS + tid;
      if (e < valid) fp_count(lo, hi, fp_classify<KB>(&ss, FpKey<KB>::okey(keys[base + e], xf), e), true);
    }
  }
  // a warp's fields stay below 2^16 (at most 512 elements): reduce the packed words, then unpack
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    lo += __shfl_xor_sync(0xFFFFFFFFu, lo, o);
    hi += __shfl_xor_sync(0xFFFFFFFFu, hi, o);
  }
  if ((tid & 31) < FP_NB) {
    const unsigned int c = fp_field(lo, hi, tid & 31);
    if (c) atomicAdd(&cnt[tid & 31], c);
  }
  __syncthreads();
  if (tid < FP_NB) {
    const unsigned int c = cnt[tid];
    tile_counts[(size_t)blockIdx.x * FP_NB + tid] = c;
    if (c) atomicAdd(&chunk_sums[(size_t)(blockIdx.x / FP_CHUNK_TILES) * FP_NB + tid], (unsigned long long)c);
  }
}

// The counting pass that also counts, per destination, the digits of every radix pass of the keys
// it will send there: the histogram pass of the receivers' local sorts, done where the keys are in
// registers anyway (the classification keeps the ALU pipe busy, the counters the shared-memory
// pipe).  One wave of CTAs, each over tiles c, c + gridDim.x, ...; the tables stay in shared
// memory over all tiles of the CTA and are added to sent_hist[(dest * KB + byte) * 256 + digit] once.
// A byte that is the same in every key of a tile (constant high bytes, sorted input) is counted from
// the tile's per-destination totals: the lanes of a warp would otherwise queue up on one counter.
template <int KB>
__global__ void __launch_bounds__(FP_THREADS)
part_count_hist_kernel(const typename FpKey<KB>::Raw* __restrict__ keys, long long n, long long ntiles, int xf,
                       const LocalSplitter* __restrict__ split, unsigned int* __restrict__ tile_counts,
                       unsigned long long* __restrict__ chunk_sums, unsigned int* __restrict__ sent_hist)
{
  using Raw = typename FpKey<KB>::Raw;
  using OK  = typename FpKey<KB>::OK;
  extern __shared__ __align__(16) unsigned char fp_count_smem[];
  unsigned int* shist = reinterpret_cast<unsigned int*>(fp_count_smem);  // FP_NB * KB * RADIX
  __shared__ FpSplit<KB> ss;
  __shared__ unsigned long long wtot[2 * FP_WARPS], wbits[2 * FP_WARPS];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int VEC = 16 / KB;         // keys per 16-byte vector
  constexpr int NV  = FP_ITEMS / VEC;  // vectors per thread
  for (int i = tid; i < FP_NB * KB * RADIX; i += FP_THREADS) shist[i] = 0;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long base = tile * FP_TILE;
    fp_load_splitters<KB>(&ss, split, base, tid);
    __syncthreads();
    const int valid = (int)min((long long)FP_TILE, n - base);
    const bool vec  = valid == FP_TILE && ((reinterpret_cast<uintptr_t>(keys + base) & 15u) == 0);
    union {
      uint4 q;
      Raw r[VEC];
    } u[NV];
    if (vec) {
      const uint4* v = reinterpret_cast<const uint4*>(keys + base);
#pragma unroll
      for (int j = 0; j < NV; ++j) u[j].q = __ldg(v + j * FP_THREADS + tid);
    } else {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const int e = (j * FP_THREADS + tid) * VEC + k;
          u[j].r[k]   = e < valid ? keys[base + e] : (Raw)0;
        }
      }
    }
    unsigned long long bs = 0, lo = 0, hi = 0;
    OK kor = 0, kand = (OK)~(OK)0;
    const bool simple = ss.simple != 0;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const int e          = (j * FP_THREADS + tid) * VEC + k;
        const OK o           = FpKey<KB>::okey(u[j].r[k], xf);
        const unsigned int b = simple ? fp_classify_simple<KB>(&ss, o) : fp_classify<KB>(&ss, o, e);
        bs |= (unsigned long long)b << (4 * (j * VEC + k));
        fp_count(lo, hi, b, e < valid);
        kor |= o;
        kand &= o;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo += __shfl_xor_sync(0xFFFFFFFFu, lo, o);
      hi += __shfl_xor_sync(0xFFFFFFFFu, hi, o);
      kor |= (OK)__shfl_xor_sync(0xFFFFFFFFu, kor, o);
      kand &= (OK)__shfl_xor_sync(0xFFFFFFFFu, kand, o);
    }
    if (lane == 0) {
      wtot[2 * warp]      = lo;
      wtot[2 * warp + 1]  = hi;
      wbits[2 * warp]     = (unsigned long long)kor;
      wbits[2 * warp + 1] = (unsigned long long)kand;
    }
    __syncthreads();
    unsigned long long tlo = 0, thi = 0, tor = 0, tand = ~0ull;
#pragma unroll
    for (int w = 0; w < FP_WARPS; ++w) {
      tlo += wtot[2 * w];
      thi += wtot[2 * w + 1];
      tor |= wbits[2 * w];
      tand &= wbits[2 * w + 1];
    }
    if (tid < FP_NB) {
      const unsigned int c = fp_field(tlo, thi, tid);
      tile_counts[(size_t)tile * FP_NB + tid] = c;
      if (c) atomicAdd(&chunk_sums[(size_t)(tile / FP_CHUNK_TILES) * FP_NB + tid], (unsigned long long)c);
    }
    const unsigned long long varying = valid == FP_TILE ? (tor ^ tand) : ~0ull;
#pragma unroll
    for (int p = 0; p < KB; ++p) {
      if ((varying >> (8 * p)) & 0xFFull) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            const int e = (j * FP_THREADS + tid) * VEC + k;
            if (e < valid) {
              const OK o           = FpKey<KB>::okey(u[j].r[k], xf);
              const unsigned int b = (unsigned int)(bs >> (4 * (j * VEC + k))) & 15u;
              atomicAdd(&shist[(b * KB + p) * RADIX + ((unsigned int)(o >> (8 * p)) & 0xFFu)], 1u);
            }
          }
        }
      } else if (tid < FP_NB) {
        const unsigned int c = fp_field(tlo, thi, tid);
        if (c) atomicAdd(&shist[(tid * KB + p) * RADIX + ((unsigned int)(tor >> (8 * p)) & 0xFFu)], c);
      }
    }
    __syncthreads();  // the splitters and the warps' words are free for the next tile
  }
  __syncthreads();
  for (int i = tid; i < FP_NB * KB * RADIX; i += FP_THREADS) {
    const unsigned int c = shist[i];
    if (c) atomicAdd(&sent_hist[i], c);
  }
}

// One CTA per chunk of tiles, one warp per destination: the chunk starts from the sums of the
// chunks before it (a short loop over chunk_sums), then its tiles get their exclusive prefixes.
// The last chunk's CTA also writes the totals.
__global__ void __launch_bounds__(FP_NB * 32)
tile_scan_fast_kernel(const unsigned int* __restrict__ tile_counts, long long ntiles, const unsigned long long* __restrict__ chunk_sums,
                      unsigned long long* __restrict__ tile_off, long long* __restrict__ totals)
{
  const int b = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long chunk = blockIdx.x, nchunks = gridDim.x;
  unsigned long long before = 0;
  for (long long c = lane; c < chunk; c += 32) before += chunk_sums[c * FP_NB + b];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xFFFFFFFFu, before, o);
  const long long t0 = chunk * FP_CHUNK_TILES;
  const long long t1 = min(t0 + FP_CHUNK_TILES, ntiles);
  unsigned long long run = before;
  for (long long t = t0; t < t1; t += 32) {
    const unsigned int c = t + lane < t1 ? tile_counts[(t + lane) * FP_NB + b] : 0u;
    unsigned int incl    = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += v;
    }
    if (t + lane < t1) tile_off[(t + lane) * FP_NB + b] = run + incl - c;
    run += __shfl_sync(0xFFFFFFFFu, incl, 31);
  }
  if (chunk == nchunks - 1 && lane == 0) totals[b] = (long long)run;
}

struct FpDst {
  void* keys[FP_NB];
  void* pay[FP_NB];
};

template <int KB, int PAYB> struct FpSmem {
  static constexpr size_t OFF_PAY   = (size_t)FP_TILE * KB;
  static constexpr size_t OFF_SPLIT = OFF_PAY + (size_t)FP_TILE * PAYB;
  static constexpr size_t OFF_WTOT  = (OFF_SPLIT + sizeof(FpSplit<KB>) + 15) / 16 * 16;  // FP_WARPS x 2 packed words
  static constexpr size_t OFF_START = OFF_WTOT + FP_WARPS * 16;                          // FP_NB + 1 tile positions
  static constexpr size_t OFF_GOFF  = (OFF_START + (FP_NB + 1) * 4 + 7) / 8 * 8;
  static constexpr size_t OFF_DKEY  = OFF_GOFF + FP_NB * 8;
  static constexpr size_t OFF_DPAY  = OFF_DKEY + FP_NB * 8;
  static constexpr size_t OFF_BAR   = OFF_DPAY + FP_NB * 8;
  static constexpr size_t OFF_POS   = (OFF_BAR + 8 + 15) / 16 * 16;    // FP_NB x FP_THREADS next places, one row per destination
  static constexpr size_t BYTES     = OFF_POS + (size_t)FP_NB * FP_THREADS * 4;
};

// Stable partition of tiles into the destinations' receive buffers (see the vote-based kernel
// of the same role for the contract).  CTA c takes tiles c, c + gridDim.x, ...; launched with one
// CTA per tile.
template <int KB, int PAYB>
__global__ void __launch_bounds__(FP_THREADS, 4)
part_scatter_fast_kernel(const typename FpKey<KB>::Raw* __restrict__ keys, long long n, int xf,
                         const LocalSplitter* __restrict__ split, const unsigned long long* __restrict__ tile_off,
                         const __grid_constant__ FpDst dst, long long global_offset, long long pay_base,
                         unsigned int* __restrict__ status)
{
  using Raw = typename FpKey<KB>::Raw;
  using OK  = typename FpKey<KB>::OK;
  using S   = FpSmem<KB, PAYB>;
  extern __shared__ __align__(128) unsigned char smem[];
  Raw* skeys               = reinterpret_cast<Raw*>(smem);
  unsigned char* spay      = smem + S::OFF_PAY;
  FpSplit<KB>* ss          = reinterpret_cast<FpSplit<KB>*>(smem + S::OFF_SPLIT);
  unsigned long long* wtot = reinterpret_cast<unsigned long long*>(smem + S::OFF_WTOT);
  unsigned int* bstart     = reinterpret_cast<unsigned int*>(smem + S::OFF_START);
  unsigned long long* goff = reinterpret_cast<unsigned long long*>(smem + S::OFF_GOFF);
  void** dkey              = reinterpret_cast<void**>(smem + S::OFF_DKEY);
  void** dpay              = reinterpret_cast<void**>(smem + S::OFF_DPAY);
  uint64_t* bar            = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  unsigned int* spos       = reinterpret_cast<unsigned int*>(smem + S::OFF_POS);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long ntiles = (n + FP_TILE - 1) / FP_TILE;
  if (tid < FP_NB) {
    dkey[tid] = dst.keys[tid];
    dpay[tid] = dst.pay[tid];
  }
  if (tid == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  uint32_t phase = 0;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long base = tile * FP_TILE;
    fp_load_splitters<KB>(ss, split, base, tid);
    if (tid < FP_NB) goff[tid] = tile_off[(size_t)tile * FP_NB + tid];
    __syncthreads();
    const int valid = (int)min((long long)FP_TILE, n - base);
    const bool vec  = valid == FP_TILE && ((reinterpret_cast<uintptr_t>(keys + base) & 15u) == 0);
    Raw key[FP_ITEMS];
    const int first = tid * FP_ITEMS;
    if (vec) {
      // the tile arrives in the staging buffer by one bulk asynchronous copy (TMA engine); every
      // thread then reads its 16 consecutive keys from shared memory
      int arrived = 1;
      if (tid == 0) {
        fence_proxy_async();  // the generic accesses of the previous tile come before the copy
        mbar_expect_tx(bar, (uint32_t)(FP_TILE * KB));
        bulk_load(skeys, keys + base, (uint32_t)(FP_TILE * KB), bar);
        arrived = mbar_wait_bounded(bar, phase);
      }
      phase ^= 1u;
      if (!__syncthreads_and(arrived)) {
        if (tid == 0) atomicMax(status, DEV_ERR_TIMEOUT);  // nothing more is written by this CTA
        return;
      }
      fp_load_keys<KB>(key, skeys, first, valid, true);
    } else {
      fp_load_keys<KB>(key, keys + base, first, valid, false);
    }

    // destinations of my elements (4 bits each) and my counts per destination
    unsigned long long bs = 0, lo = 0, hi = 0;
    if (ss->simple) {  // the same for the whole CTA
#pragma unroll
      for (int i = 0; i < FP_ITEMS; ++i) {
        const OK o           = FpKey<KB>::okey(key[i], xf);
        const unsigned int b = fp_classify_simple<KB>(ss, o);
        bs |= (unsigned long long)b << (4 * i);
        fp_count(lo, hi, b, first + i < valid);
      }
    } else {
#pragma unroll
      for (int i = 0; i < FP_ITEMS; ++i) {
        const OK o           = FpKey<KB>::okey(key[i], xf);
        const unsigned int b = fp_classify<KB>(ss, o, first + i);
        bs |= (unsigned long long)b << (4 * i);
        fp_count(lo, hi, b, first + i < valid);
      }
    }
    // exclusive prefix of the packed counts over the threads of the CTA (fields stay below 2^16)
    unsigned long long ilo = lo, ihi = hi;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long a = __shfl_up_sync(0xFFFFFFFFu, ilo, o);
      const unsigned long long c = __shfl_up_sync(0xFFFFFFFFu, ihi, o);
      if (lane >= o) {
        ilo += a;
        ihi += c;
      }
    }
    if (lane == 31) {
      wtot[2 * warp]     = ilo;
      wtot[2 * warp + 1] = ihi;
    }
    __syncthreads();
    unsigned long long plo = ilo - lo, phi = ihi - hi, tlo = 0, thi = 0;
#pragma unroll
    for (int w = 0; w < FP_WARPS; ++w) {
      const unsigned long long a = wtot[2 * w], c = wtot[2 * w + 1];
      if (w < warp) {
        plo += a;
        phi += c;
      }
      tlo += a;
      thi += c;
    }
    // start of every destination's piece in the staged tile: inclusive prefix over the fields by one
    // multiplication (no field overflows: a tile holds fewer than 2^16 elements), minus the counts
    const unsigned long long inc_lo = tlo * FP_ONES;
    const unsigned long long inc_hi = thi * FP_ONES + (inc_lo >> 48) * FP_ONES;
    plo += inc_lo - tlo;
    phi += inc_hi - thi;
    if (tid == 0) {
#pragma unroll
      for (int b = 0; b < FP_NB; ++b) bstart[b] = fp_field(inc_lo - tlo, inc_hi - thi, b);
      bstart[FP_NB] = (unsigned int)valid;
    }
    // stage: position = start of the destination's piece + elements of lower threads + my earlier
    // ones.  The thread's next place per destination lives in its own column of a small table in
    // shared memory (column = thread = bank: no conflicts, and nobody else touches it): a load, an add
    // and a store per element instead of field arithmetic on the packed 64-bit words.
    unsigned int* my_pos = spos + tid;
#pragma unroll
    for (int b = 0; b < FP_NB; ++b) my_pos[b * FP_THREADS] = fp_field(plo, phi, b);
    const long long g0 = global_offset + base + first;
    const uint32_t g32 = (uint32_t)(g0 - pay_base);
#pragma unroll
    for (int i = 0; i < FP_ITEMS; ++i) {
      const unsigned int b = (unsigned int)(bs >> (4 * i)) & 15u;
      if (first + i < valid) {
        unsigned int* q      = my_pos + b * FP_THREADS;
        const unsigned int p = *q;
        *q                   = p + 1;
        skeys[p]             = key[i];
        if (PAYB == 4) reinterpret_cast<uint32_t*>(spay)[p] = g32 + (uint32_t)i;
        if (PAYB == 8) reinterpret_cast<int64_t*>(spay)[p] = (int64_t)(g0 + i);
      }
    }
    __syncthreads();
    // copy-out, one destination after the other: a warp stores groups of 32 consecutive elements
    // that start on 32-element boundaries OF THE DESTINATION, so that every store instruction fills
    // whole 128-byte lines there (the pieces start wherever the counts put them).  Over NVLink a
    // line written in two parts costs two packets.
#pragma unroll 1
    for (int b = 0; b < FP_NB; ++b) {
      const int s0 = (int)bstart[b], len = (int)bstart[b + 1] - s0;
      if (len <= 0) continue;
      Raw* kdst            = static_cast<Raw*>(dkey[b]) + goff[b];
      const int mis        = (int)((reinterpret_cast<uintptr_t>(kdst) / KB) & 31u);
      const int groups     = (len + mis + 31) >> 5;
      unsigned char* pdst  = PAYB ? static_cast<unsigned char*>(dpay[b]) + goff[b] * PAYB : nullptr;
      for (int g = warp; g < groups; g += FP_WARPS) {
        const int i = (g << 5) + lane - mis;
        if (i >= 0 && i < len) {
          kdst[i] = skeys[s0 + i];
          if (PAYB == 4) reinterpret_cast<uint32_t*>(pdst)[i] = reinterpret_cast<const uint32_t*>(spay)[s0 + i];
          if (PAYB == 8) reinterpret_cast<int64_t*>(pdst)[i] = reinterpret_cast<const int64_t*>(spay)[s0 + i];
        }
      }
    }
    __syncthreads();  // the tile's tables and staging buffers are free for the next tile
  }
}

// Hands every destination the digit counts of what this rank sent it: block d stores
// sent_hist[d] ([KB][RADIX]) into destination d's landing area, slot `my_rank`.
__global__ void hist_deliver_kernel(const unsigned int* __restrict__ sent_hist, const __grid_constant__ FpDst landing, int kb,
                                    int my_rank)
{
  unsigned int* dst = static_cast<unsigned int*>(landing.keys[blockIdx.x]);
  if (dst == nullptr) return;
  dst += (size_t)my_rank * kb * RADIX;
  const unsigned int* src = sent_hist + (size_t)blockIdx.x * kb * RADIX;
  for (int i = threadIdx.x; i < kb * RADIX; i += blockDim.x) dst[i] = src[i];
}

}  // namespace b2s
