// Stable k-way merge of the sorted runs a rank receives in the exchange (one run per source
// rank, in rank order): one pass over the data instead of the reference's log2(P) sweeps of
// pairwise thrust::merge (src/cupynumeric/sort/sort.cu:608-790).
//
// Kernel A finds, for every output tile boundary, where that boundary cuts each run (one warp
// per boundary, one lane per run, bisection on the key value).  Kernel B loads a tile's pieces
// into shared memory and merges them there with a tree of pairwise merge-path merges.
#pragma once
#include "b2s_common.cuh"

namespace b2s {

constexpr int MERGE_MAX_RUNS = 32;
constexpr int MERGE_THREADS  = 256;
constexpr int MERGE_VT       = 8;
constexpr int MERGE_TILE     = MERGE_THREADS * MERGE_VT;

struct MergeRuns {
  const void* keys[MERGE_MAX_RUNS];     // run i: len[i] sorted keys
  const void* idx[MERGE_MAX_RUNS];      // payload of run i (argsort) or null
  long long idx_base[MERGE_MAX_RUNS];   // added to a 32-bit payload
  int idx_bytes[MERGE_MAX_RUNS];        // payload width of run i: 8 (int64) or 4 (uint32 + idx_base)
  long long len[MERGE_MAX_RUNS];
  int nruns;
};

template <int KB>
__device__ __forceinline__ unsigned long long okey_at(const void* base, long long i, int xf)
{
  using K = typename KeyOf<KB>::type;
  return (unsigned long long)to_ordered_rt<KB>(static_cast<const K*>(base)[i], xf);
}

// first position in [lo, hi) of run whose ordered key is >= x
template <int KB>
__device__ __forceinline__ long long lower_bound_okey(const void* base, long long lo, long long hi,
                                                      unsigned long long x, int xf)
{
  while (lo < hi) {
    const long long mid = lo + ((hi - lo) >> 1);
    if (okey_at<KB>(base, mid, xf) < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// The same search with ARY - 1 probes per step.  The probes of a step are independent loads, so a
// step costs one memory latency like a step of the binary search, and there are log2(ARY) times
// fewer steps: the searches of the partition kernel are chains of dependent loads and nothing else.
template <int KB, int ARY>
__device__ __forceinline__ long long lower_bound_okey_wide(const void* base, long long lo, long long hi,
                                                           unsigned long long x, int xf)
{
  static_assert(ARY >= 2 && (ARY & (ARY - 1)) == 0, "ARY must be a power of two");
  constexpr int SH = ARY == 2 ? 1 : ARY == 4 ? 2 : ARY == 8 ? 3 : 4;
  while (hi - lo >= ARY) {
    const long long span = hi - lo;
    int c = 0;  // probes with key < x; the keys are sorted, so these are the first c probes
#pragma unroll
    for (int j = 1; j < ARY; ++j) c += okey_at<KB>(base, lo + ((span * j) >> SH), xf) < x ? 1 : 0;
    const long long nlo = c == 0 ? lo : lo + ((span * c) >> SH) + 1;
    const long long nhi = c == ARY - 1 ? hi : lo + ((span * (c + 1)) >> SH);
    lo = nlo;
    hi = nhi;
  }
  int c = 0;
#pragma unroll
  for (int j = 0; j < ARY - 1; ++j) c += (lo + j < hi && okey_at<KB>(base, lo + j, xf) < x) ? 1 : 0;
  return lo + c;
}

// cuts[b * nruns + i] = number of elements of run i among the first b * MERGE_TILE elements of
// the stable merge; b = 0 .. ntiles.
//
// Two launches: the first handles every `stride`-th boundary (coarse == nullptr) and searches
// the whole runs; the second handles all boundaries and searches only between the two coarse
// cuts that enclose each one, where both the index range and the key range are narrow.
template <int KB, int ARY>
__global__ void __launch_bounds__(256)
merge_partition_kernel(MergeRuns runs, long long total, long long ntiles, int xf, long long* __restrict__ cuts,
                       long long stride, int fine)
{
  // A warp is split into groups of gw lanes (gw = run count rounded up to a power of two); each
  // group finds one boundary, one lane per run.  All groups run the same number of loop trips so
  // that the warp stays converged for the shuffles.
  const int nruns = runs.nruns;
  int gw = 1;
  while (gw < nruns) gw <<= 1;
  const int groups    = 32 / gw;
  const int lane      = threadIdx.x & 31;
  const int sub       = lane / gw, run = lane % gw;
  const long long w   = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * groups + sub;
  long long b         = 0;
  bool live           = true;
  if (!fine) {
    // coarse boundaries: 0, stride, 2*stride, ..., and ntiles itself
    const long long ncoarse = (ntiles + stride - 1) / stride + 1;
    live = w < ncoarse;
    b    = w * stride < ntiles ? w * stride : ntiles;
  } else {
    live = w <= ntiles;
    b    = w;
    if (live && (b % stride == 0 || b == ntiles)) live = false;  // written by the coarse launch
  }
  const bool mine     = live && run < nruns;
  const long long n_i = mine ? runs.len[run] : 0;
  const void* base    = mine ? runs.keys[run] : nullptr;
  long long r         = b * MERGE_TILE;
  if (r > total) r = total;
  const bool search   = live && r > 0 && r < total;

  long long lo = 0, hi = search ? n_i : 0;  // this run's cut lies in [lo, hi]
  if (search && fine && mine) {
    const long long c0 = (b / stride) * stride;
    const long long c1 = c0 + stride < ntiles ? c0 + stride : ntiles;
    lo                 = cuts[c0 * nruns + run];
    hi                 = cuts[c1 * nruns + run];
  }
  const long long hi0 = hi;
  constexpr int BITS  = 8 * KB;
  // Bits above the highest one in which the smallest and the largest key of the searched ranges
  // differ are common to every candidate: the bisection starts below them.
  unsigned long long kmin = ~0ull, kmax = 0;
  if (hi > lo) {
    kmin = okey_at<KB>(base, lo, xf);
    kmax = okey_at<KB>(base, hi - 1, xf);
  }
  for (int s = gw >> 1; s > 0; s >>= 1) {
    const unsigned long long a = __shfl_xor_sync(0xFFFFFFFFu, kmin, s);
    const unsigned long long c = __shfl_xor_sync(0xFFFFFFFFu, kmax, s);
    kmin = a < kmin ? a : kmin;
    kmax = c > kmax ? c : kmax;
  }
  const unsigned long long diff = kmax >= kmin ? (kmin ^ kmax) : 0ull;
  const int top = diff ? 63 - __clzll((long long)diff) : -1;  // highest varying bit
  // v = key of the r-th element of the merge = max{x : #(keys < x) <= r}, built bit by bit.
  unsigned long long x = top >= 63 ? 0ull : (top < 0 ? kmin : (kmin >> (top + 1)) << (top + 1));
  for (int bit = BITS - 1; bit >= 0; --bit) {
    const bool step               = search && bit <= top;
    const unsigned long long cand = x | (1ull << bit);
    const long long p = step ? lower_bound_okey_wide<KB, ARY>(base, lo, hi, cand, xf) : 0;
    long long less    = p;
    for (int s = gw >> 1; s > 0; s >>= 1) less += __shfl_xor_sync(0xFFFFFFFFu, less, s);
    if (step) {
      if (less <= r) {
        x  = cand;
        lo = p;
      } else {
        hi = p;
      }
    }
  }
  // lo = #(keys < v) in this run (clamped to the searched range); ties (== v) go out in run order
  const long long lower = lo;
  long long upper       = hi0;
  if (search && x != (BITS == 64 ? ~0ull : ((1ull << (BITS & 63)) - 1)))
    upper = lower_bound_okey_wide<KB, ARY>(base, lo, hi0, x + 1, xf);
  long long less_total = lower;
  for (int s = gw >> 1; s > 0; s >>= 1) less_total += __shfl_xor_sync(0xFFFFFFFFu, less_total, s);
  const long long equal = upper - lower;
  long long incl        = equal;  // inclusive prefix of `equal` over the group's lanes
  for (int s = 1; s < gw; s <<= 1) {
    const long long t = __shfl_up_sync(0xFFFFFFFFu, incl, s, gw);
    if (run >= s) incl += t;
  }
  long long take = (r - less_total) - (incl - equal);  // ties left for this run
  take           = take < 0 ? 0 : (take > equal ? equal : take);
  long long cut  = lower + take;
  if (r == 0) cut = 0;
  if (r == total) cut = mine ? runs.len[run] : 0;
  if (mine) cuts[b * nruns + run] = cut;
}

constexpr long long MERGE_COARSE_STRIDE = 64;

// Shared-memory index of logical position i in the merge buffers.  A thread works on
// MERGE_VT consecutive positions, so unpadded accesses of a warp would fall on two banks; one
// spare slot per eight spreads them over all banks.
__device__ __host__ __forceinline__ constexpr int mpad(int i) { return i + (i >> 3); }
constexpr int MERGE_PADDED = MERGE_TILE + MERGE_TILE / 8 + 8;

// FLT: float keys, whose ordered image cannot be mapped back (NaN payloads, signed zeros).
// Slots (the position a merged element had when it was loaded) are carried only when something
// has to be fetched through them afterwards: the payload (ARGS) or the raw float key (FLT).
// Plain integer key merges move nothing but the ordered keys and map them back on the way out.
template <int KB, bool ARGS, bool FLT>
struct MergeSmem {
  static constexpr bool SLOTS = ARGS || FLT;
  static constexpr bool RAW   = FLT && !ARGS;
  // keys of at most 32 bits share a 64-bit word with their slot: (ordered key << 32) | slot.
  // Comparing the words orders by key, then by slot, which is run order: the merge stays stable
  // and needs no separate slot arrays.
  static constexpr bool PACK  = SLOTS && KB <= 4;
  // merge-buffer entry: 4 bytes for plain integer keys of at most 32 bits, else 8
  static constexpr size_t WB       = (!SLOTS && KB <= 4) ? 4 : 8;
  static constexpr size_t OFF_RAW  = 0;
  static constexpr size_t OFF_OK0  = (RAW ? ((size_t)MERGE_TILE * KB + 15) / 16 * 16 : 0);
  static constexpr size_t OFF_OK1  = OFF_OK0 + (size_t)MERGE_PADDED * WB;
  static constexpr size_t OFF_SL0  = OFF_OK1 + (size_t)MERGE_PADDED * WB;
  static constexpr size_t OFF_SL1  = OFF_SL0 + ((SLOTS && !PACK) ? (size_t)MERGE_PADDED * 2 : 0);
  static constexpr size_t OFF_BND  = (OFF_SL1 + ((SLOTS && !PACK) ? (size_t)MERGE_PADDED * 2 : 0) + 15) / 16 * 16;
  static constexpr size_t OFF_SRC  = (OFF_BND + (MERGE_MAX_RUNS + 1) * 4 + 15) / 16 * 16;  // 8-byte entries
  static constexpr size_t OFF_KP   = OFF_SRC + MERGE_MAX_RUNS * 8;   // run key pointers
  static constexpr size_t OFF_IP   = OFF_KP + MERGE_MAX_RUNS * 8;    // run payload pointers
  static constexpr size_t OFF_IB   = OFF_IP + MERGE_MAX_RUNS * 8;    // payload bases (negative: int64 payload)
  static constexpr size_t BYTES    = OFF_IB + MERGE_MAX_RUNS * 8;
};

template <size_t B> struct MergeWord { using type = unsigned long long; };
template <> struct MergeWord<4> { using type = uint32_t; };

// inverse of to_ordered for the integer orderings
template <int KB>
__device__ __forceinline__ typename KeyOf<KB>::type from_ordered_int(unsigned long long o, int xf)
{
  using K        = typename KeyOf<KB>::type;
  constexpr K SB = (K)((K)1 << (8 * KB - 1));
  return xf == XF_SIGNED ? (K)((K)o ^ SB) : (K)o;
}

// One CTA per output tile.  ARGS: emit the int64 payload (argsort); else emit the keys.
template <int KB, bool ARGS, bool FLT>
__global__ void __launch_bounds__(MERGE_THREADS)
merge_tiles_kernel(MergeRuns runs, long long total, int xf, const long long* __restrict__ cuts,
                   void* __restrict__ out)
{
  using K = typename KeyOf<KB>::type;
  using S = MergeSmem<KB, ARGS, FLT>;
  constexpr bool PACK  = S::PACK;
  constexpr bool SLOTS = S::SLOTS && !PACK;  // separate slot arrays
  constexpr bool RAW   = S::RAW;
  extern __shared__ __align__(16) unsigned char smem[];
  K* raw                    = reinterpret_cast<K*>(smem + S::OFF_RAW);
  using W                   = typename MergeWord<S::WB>::type;
  W* ok[2]                  = {reinterpret_cast<W*>(smem + S::OFF_OK0), reinterpret_cast<W*>(smem + S::OFF_OK1)};
  unsigned short* sl[2]     = {reinterpret_cast<unsigned short*>(smem + S::OFF_SL0),
                               reinterpret_cast<unsigned short*>(smem + S::OFF_SL1)};
  int* bnd                  = reinterpret_cast<int*>(smem + S::OFF_BND);        // piece starts in the tile
  long long* src0           = reinterpret_cast<long long*>(smem + S::OFF_SRC);  // piece starts in the runs
  const K** kptr            = reinterpret_cast<const K**>(smem + S::OFF_KP);
  const void** iptr         = reinterpret_cast<const void**>(smem + S::OFF_IP);
  long long* ibase          = reinterpret_cast<long long*>(smem + S::OFF_IB);

  const int tid        = threadIdx.x;
  const long long b    = blockIdx.x;
  const int nruns      = runs.nruns;
  const long long base = b * MERGE_TILE;
  const int count      = (int)((total - base) < MERGE_TILE ? (total - base) : MERGE_TILE);
  int p2 = 1;
  while (p2 < nruns) p2 <<= 1;  // tree width

  // run descriptors go to shared memory: indexing kernel parameters with a run-time index would
  // make the compiler spill the whole parameter block to local memory
  if (tid < MERGE_MAX_RUNS) {
    kptr[tid] = tid < nruns ? static_cast<const K*>(runs.keys[tid]) : nullptr;
    iptr[tid] = tid < nruns ? runs.idx[tid] : nullptr;
    // a 32-bit payload is a position below 2^32 plus a non-negative base; -1 marks int64 payloads
    ibase[tid] = (tid < nruns && runs.idx_bytes[tid] == 4) ? runs.idx_base[tid] : -1;
  }
  if (tid == 0) {
    int off = 0;
    for (int i = 0; i < nruns; ++i) {
      const long long c0 = cuts[b * nruns + i], c1 = cuts[(b + 1) * nruns + i];
      bnd[i]  = off;
      src0[i] = c0;
      off += (int)(c1 - c0);
    }
    for (int i = nruns; i <= p2; ++i) bnd[i] = off;  // padding runs are empty
  }
  __syncthreads();

  // load the pieces, run after run (coalesced inside a run)
  for (int i = 0; i < nruns; ++i) {
    const int q0 = bnd[i], q1 = bnd[i + 1];
    const K* kp  = kptr[i] + src0[i];
    for (int q = q0 + tid; q < q1; q += MERGE_THREADS) {
      const K k = kp[q - q0];
      if (RAW) raw[q] = k;
      const unsigned long long o = (unsigned long long)to_ordered_rt<KB>(k, xf);
      ok[0][mpad(q)] = PACK ? (W)((o << 32) | (unsigned long long)q) : (W)o;
      if (SLOTS) sl[0][mpad(q)] = (unsigned short)q;
    }
  }
  __syncthreads();

  // tree of pairwise stable merges; ties take from the lower run first
  int cur = 0;
  for (int g = 2; g <= p2; g <<= 1) {
    const W* ik              = ok[cur];
    const unsigned short* is = sl[cur];
    W* okd                   = ok[cur ^ 1];
    unsigned short* sld          = sl[cur ^ 1];
    int q        = tid * MERGE_VT;
    const int q1 = min(q + MERGE_VT, count);
    int pair     = 0;
    while (q < q1) {
      while (bnd[(pair + 1) * g] <= q) ++pair;  // pair whose output span holds q
      const int s0 = bnd[pair * g], mid = bnd[pair * g + g / 2], s1 = bnd[(pair + 1) * g];
      const int na = mid - s0, nb = s1 - mid;
      const int end = min(q1, s1);
      const int diag = q - s0;
      int lo = max(0, diag - nb), hi = min(diag, na);
      while (lo < hi) {
        const int m = (lo + hi) >> 1;
        if (ik[mpad(s0 + m)] <= ik[mpad(mid + diag - 1 - m)]) lo = m + 1; else hi = m;
      }
      int ia = s0 + lo, ib = mid + diag - lo;  // absolute read positions in the two runs
      constexpr W INF = (W)~(W)0;
      W ka = ia < mid ? ik[mpad(ia)] : INF, kb = ib < s1 ? ik[mpad(ib)] : INF;
#pragma unroll
      for (int j = 0; j < MERGE_VT; ++j) {
        if (q < end) {
          // an exhausted run reads as +inf; on equal keys the lower run wins unless it is exhausted
          const bool take_a = ib >= s1 || (ia < mid && ka <= kb);
          const int from    = take_a ? ia : ib;
          okd[mpad(q)]      = take_a ? ka : kb;
          if (SLOTS) sld[mpad(q)] = is[mpad(from)];
          ia += take_a ? 1 : 0;
          ib += take_a ? 0 : 1;
          const int nxt              = take_a ? ia : ib;
          const bool live            = take_a ? (ia < mid) : (ib < s1);
          const W v                  = live ? ik[mpad(nxt)] : INF;
          ka = take_a ? v : ka;
          kb = take_a ? kb : v;
          ++q;
        }
      }
    }
    cur ^= 1;
    __syncthreads();
  }

  const unsigned short* fs     = sl[cur];
  const W* fp                  = ok[cur];
  auto slot_of = [&](int q) -> unsigned int { return PACK ? (unsigned int)(fp[mpad(q)] & 0xFFFFu) : (unsigned int)fs[mpad(q)]; };
  if (ARGS) {
    // the merge buffer that is no longer read becomes the payload staging area
    int64_t* pay = reinterpret_cast<int64_t*>(ok[cur ^ 1]);
    for (int i = 0; i < nruns; ++i) {
      const int q0 = bnd[i], q1 = bnd[i + 1];
      const long long ib = ibase[i];
      if (ib < 0) {
        const int64_t* ip = static_cast<const int64_t*>(iptr[i]) + src0[i];
        for (int q = q0 + tid; q < q1; q += MERGE_THREADS) pay[q] = ip[q - q0];
      } else {
        const uint32_t* ip = static_cast<const uint32_t*>(iptr[i]) + src0[i];
        for (int q = q0 + tid; q < q1; q += MERGE_THREADS) pay[q] = (int64_t)ip[q - q0] + ib;
      }
    }
    __syncthreads();
    int64_t* o = static_cast<int64_t*>(out) + base;
    for (int q = tid; q < count; q += MERGE_THREADS) o[q] = pay[slot_of(q)];
  } else if (RAW) {
    K* o = static_cast<K*>(out) + base;
    for (int q = tid; q < count; q += MERGE_THREADS) o[q] = raw[slot_of(q)];
  } else {
    K* o                         = static_cast<K*>(out) + base;
    const W* fk                  = ok[cur];
    for (int q = tid; q < count; q += MERGE_THREADS) o[q] = from_ordered_int<KB>(fk[mpad(q)], xf);
  }
}

}  // namespace b2s
