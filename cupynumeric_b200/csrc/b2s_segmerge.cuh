// Segmented sort of rows that fit in shared memory, by a stable merge sort: every thread sorts 16
// consecutive elements in registers, then log2(threads) rounds of pairwise merge-path merges run
// in one shared-memory buffer.  The cost does not depend on how many key bytes vary, which is
// what makes it the faster on-chip method for 4- and 8-byte keys (an 8-bit radix ranking pass
// costs about as much as six merge rounds).  HBM traffic is one read and one write per element.
// Stands, like the on-chip radix kernel beside it, for cub::DeviceSegmentedRadixSort and the
// short-segment thrust sort (src/cupynumeric/sort/cub_sort.cuh:73-107,145-184,
// src/cupynumeric/sort/thrust_sort.cuh:61-123).
//
// Keys are merged as their order-preserving unsigned images (to_ordered).  For floats that image
// folds -0.0 onto +0.0 and every NaN onto one value, so that the stable merge leaves them in input
// order; the way back yields +0.0 and the canonical quiet NaN, and a row that held a -0.0 or
// another NaN pattern gets those elements rewritten from the input, in input order, afterwards.
#pragma once

#include "b2s_common.cuh"

namespace b2s {

#ifndef B2S_SM_VT
#define B2S_SM_VT 16
#endif
// registers per thread the compiler may use (bounds the CTAs per SM: 65536 / (threads * this))
#ifndef B2S_SM_REGS
#define B2S_SM_REGS 64
#endif
constexpr int SM_VT = B2S_SM_VT;  // elements per thread

// shared-memory index of logical position i: one spare slot per 16 keeps a warp's blocked accesses
// (stride 16) off a single bank
__device__ __host__ __forceinline__ constexpr int smpad(int i) { return i + (i >> 4); }
static_assert(SM_VT == 16 || SM_VT == 8, "the padding rule assumes 8 or 16 elements per thread");

template <int KB> struct SmWord { using type = unsigned long long; };
template <> struct SmWord<4> { using type = unsigned int; };

// inverse of to_ordered: integers exactly; floats up to the folding described above
template <int KB>
__device__ __forceinline__ typename KeyOf<KB>::type sm_from_ordered(typename KeyOf<KB>::type o, int xf)
{
  using K        = typename KeyOf<KB>::type;
  constexpr K SB = (K)((K)1 << (8 * KB - 1));
  if (xf == XF_UNSIGNED) return o;
  if (xf == XF_SIGNED) return (K)(o ^ SB);
  constexpr K QNAN = KB == 4 ? (K)0x7FC00000u : (K)0x7FF8000000000000ull;
  if (o == (K)~(K)0) return QNAN;
  return (o & SB) ? (K)(o ^ SB) : (K)~o;
}

// rows whose float keys need the rewrite: a -0.0, or a NaN that is not the canonical quiet NaN
template <int KB>
__device__ __forceinline__ bool sm_is_special(typename KeyOf<KB>::type raw, int xf)
{
  using K = typename KeyOf<KB>::type;
  if (xf != XF_FLOAT) return false;
  constexpr K SB   = (K)((K)1 << (8 * KB - 1));
  constexpr K EXP  = KB == 4 ? (K)0x7F800000u : (K)0x7FF0000000000000ull;
  constexpr K QNAN = KB == 4 ? (K)0x7FC00000u : (K)0x7FF8000000000000ull;
  const K mag      = (K)(raw & (K)~SB);
  return raw == SB || (mag > EXP && raw != QNAN);
}
template <int KB>
__device__ __forceinline__ bool sm_is_zero(typename KeyOf<KB>::type raw)
{
  using K = typename KeyOf<KB>::type;
  return (K)(raw << 1) == 0;
}
template <int KB>
__device__ __forceinline__ bool sm_is_nan(typename KeyOf<KB>::type raw)
{
  using K         = typename KeyOf<KB>::type;
  constexpr K SB  = (K)((K)1 << (8 * KB - 1));
  constexpr K EXP = KB == 4 ? (K)0x7F800000u : (K)0x7FF0000000000000ull;
  return (K)(raw & (K)~SB) > EXP;
}

template <int KB, bool PAIRS, int THREADS> struct SegMergeSmem {
  static constexpr int TILE   = THREADS * SM_VT;
  static constexpr int PADDED = TILE + TILE / 16 + 1;
  // 4-byte keys with payload travel as one 64-bit word (image << 32 | position); 8-byte keys with
  // payload keep the positions in a 16-bit array beside the images
  static constexpr bool PACK   = PAIRS && KB == 4;
  static constexpr bool SIDE   = PAIRS && KB == 8;
  static constexpr size_t WB   = (KB == 8 || PACK) ? 8 : 4;
  static constexpr size_t OFF_PAY  = ((size_t)PADDED * WB + 15) / 16 * 16;
  static constexpr size_t OFF_MISC = (OFF_PAY + (SIDE ? (size_t)PADDED * 2 : 0) + 15) / 16 * 16;
  static constexpr size_t BYTES    = OFF_MISC + 64 + (THREADS / 32) * 8;
};

// One CTA sorts one row at a time (grid-stride over rows); seg_len <= THREADS * 16.
template <int KB, bool PAIRS, int THREADS>
__global__ void __launch_bounds__(THREADS, (65536 / (B2S_SM_REGS * THREADS) < 1 ? 1 : (65536 / (B2S_SM_REGS * THREADS) > 16 ? 16 : 65536 / (B2S_SM_REGS * THREADS))))
segmerge_kernel(const typename KeyOf<KB>::type* __restrict__ in, typename KeyOf<KB>::type* __restrict__ out,
                int64_t* __restrict__ idx_out, unsigned int seg_len, unsigned long long nseg, int xf, int64_t index_offset)
{
  using K = typename KeyOf<KB>::type;
  using S = SegMergeSmem<KB, PAIRS, THREADS>;
  using W = typename SmWord<S::WB>::type;
  constexpr int TILE  = S::TILE;
  constexpr int WARPS = THREADS / 32;
  constexpr bool PACK = S::PACK, SIDE = S::SIDE;
  extern __shared__ __align__(16) unsigned char smem[];
  W* sw                  = reinterpret_cast<W*>(smem);
  unsigned short* sp     = reinterpret_cast<unsigned short*>(smem + S::OFF_PAY);
  unsigned int* misc     = reinterpret_cast<unsigned int*>(smem + S::OFF_MISC);   // [0..3] block bounds
  unsigned int* wsum     = misc + 16;                                             // per-warp counts of the rewrite

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int first = tid * SM_VT;
  constexpr W WMAX = (W)~(W)0;

  for (unsigned long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
    const K* src = in + seg * seg_len;
    // ---- load: coalesced into shared memory as images, then 16 consecutive ones per thread ----
    int special = 0;
    for (int e = tid; e < TILE; e += THREADS) {
      W w = WMAX;
      if ((unsigned int)e < seg_len) {
        const K raw = src[e];
        special |= sm_is_special<KB>(raw, xf) ? 1 : 0;
        const K o = to_ordered_rt<KB>(raw, xf);
        w         = PACK ? (W)(((unsigned long long)o << 32) | (unsigned int)e) : (W)o;
      }
      sw[smpad(e)] = w;
    }
    special = __syncthreads_or(special);
    W key[SM_VT];
    unsigned int pay[SIDE ? SM_VT : 1];
#pragma unroll
    for (int j = 0; j < SM_VT; ++j) {
      key[j] = sw[smpad(first + j)];
      if (SIDE) pay[j] = first + j;
    }
    // ---- stable sort of my 16 elements: odd-even transposition, swaps only on strict order ----
#pragma unroll
    for (int round = 0; round < SM_VT; ++round) {
#pragma unroll
      for (int j = round & 1; j + 1 < SM_VT; j += 2) {
        const bool sw_ = key[j + 1] < key[j];
        const W a = key[j], b = key[j + 1];
        key[j]     = sw_ ? b : a;
        key[j + 1] = sw_ ? a : b;
        if (SIDE) {
          const unsigned int pa = pay[j], pb = pay[j + 1];
          pay[j]     = sw_ ? pb : pa;
          pay[j + 1] = sw_ ? pa : pb;
        }
      }
    }
    __syncthreads();  // everybody holds its elements: the buffer may be rewritten
#pragma unroll
    for (int j = 0; j < SM_VT; ++j) {
      sw[smpad(first + j)] = key[j];
      if (SIDE) sp[smpad(first + j)] = (unsigned short)pay[j];
    }
    __syncthreads();
    // ---- merge rounds: runs of `run` elements, pairwise; my 16 outputs start at `first` ----
    for (int run = SM_VT; run < TILE; run <<= 1) {
      const int pbase = first & ~(2 * run - 1);
      const int diag  = first - pbase;
      const int a0 = pbase, b0 = pbase + run;
      int lo = max(0, diag - run), hi = min(diag, run);
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (sw[smpad(a0 + mid)] <= sw[smpad(b0 + diag - 1 - mid)]) lo = mid + 1; else hi = mid;
      }
      int ia = lo, ib = diag - lo;
      W ka = ia < run ? sw[smpad(a0 + ia)] : WMAX, kb = ib < run ? sw[smpad(b0 + ib)] : WMAX;
#pragma unroll
      for (int j = 0; j < SM_VT; ++j) {
        // an exhausted run never wins; on equal images the lower run goes first
        const bool take_a = ib >= run || (ia < run && ka <= kb);
        key[j]            = take_a ? ka : kb;
        if (SIDE) pay[j] = sp[smpad(take_a ? a0 + ia : b0 + ib)];
        ia += take_a ? 1 : 0;
        ib += take_a ? 0 : 1;
        const int nxt = take_a ? a0 + ia : b0 + ib;
        const bool ok = take_a ? ia < run : ib < run;
        const W v     = ok ? sw[smpad(nxt)] : WMAX;
        ka = take_a ? v : ka;
        kb = take_a ? kb : v;
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < SM_VT; ++j) {
        sw[smpad(first + j)] = key[j];
        if (SIDE) sp[smpad(first + j)] = (unsigned short)pay[j];
      }
      __syncthreads();
    }

    // ---- rows with -0.0 or unusual NaNs (sorts of keys): the elements the image folded are
    // fetched from the input in input order, to be written over their blocks after the store ----
    K fix_raw[SM_VT];
    int fix_at[SM_VT];
    int nfix = 0;
    if (!PAIRS && special) {
      if (tid == 0) {
        // block of zeros [z0, z1) and start of the NaN block in the sorted images
        const W zimg = (W)to_ordered_rt<KB>((K)0, xf);
        int a = 0, b = (int)seg_len;
        while (a < b) { const int m = (a + b) >> 1; if (sw[smpad(m)] < zimg) a = m + 1; else b = m; }
        misc[0] = a;
        a = 0; b = (int)seg_len;
        while (a < b) { const int m = (a + b) >> 1; if (sw[smpad(m)] < WMAX) a = m + 1; else b = m; }
        misc[1] = a;
      }
      // my 16 consecutive input elements: how many zeros / NaNs come before them
      unsigned int cz = 0, cn = 0;
      K raw[SM_VT];
#pragma unroll
      for (int j = 0; j < SM_VT; ++j) {
        raw[j] = (unsigned int)(first + j) < seg_len ? src[first + j] : (K)1;
        cz += sm_is_zero<KB>(raw[j]) ? 1u : 0u;
        cn += sm_is_nan<KB>(raw[j]) ? 1u : 0u;
      }
      unsigned int packed = cz | (cn << 16), incl = packed;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane == 31) wsum[warp] = incl;
      __syncthreads();
      unsigned int before = incl - packed;
      for (int w = 0; w < warp; ++w) before += wsum[w];
      int rz = (int)(before & 0xFFFFu) + (int)misc[0], rn = (int)(before >> 16) + (int)misc[1];
#pragma unroll
      for (int j = 0; j < SM_VT; ++j) {
        const bool z = sm_is_zero<KB>(raw[j]), nn = sm_is_nan<KB>(raw[j]);
        if (z || nn) {
          fix_raw[nfix] = raw[j];
          fix_at[nfix]  = z ? rz : rn;
          ++nfix;
        }
        rz += z ? 1 : 0;
        rn += nn ? 1 : 0;
      }
    }

    // ---- store (coalesced) ----
    K* dst = out ? out + seg * seg_len : nullptr;
    if (!PAIRS) {
      for (int e = tid; e < (int)seg_len; e += THREADS) dst[e] = sm_from_ordered<KB>((K)sw[smpad(e)], xf);
      if (special) {
        __syncthreads();  // the plain store of the row is complete
        for (int f = 0; f < nfix; ++f) dst[fix_at[f]] = fix_raw[f];
      }
    } else {
      int64_t* idst = idx_out + seg * seg_len;
      if (dst != nullptr) {
        // keys as well: fetched through the positions before anything of the row is written
        // (the output may be the input)
        K kraw[SM_VT];
#pragma unroll
        for (int j = 0; j < SM_VT; ++j) {
          const int e = j * THREADS + tid;
          if (e < (int)seg_len) kraw[j] = src[PACK ? (unsigned int)sw[smpad(e)] : (unsigned int)sp[smpad(e)]];
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < SM_VT; ++j) {
          const int e = j * THREADS + tid;
          if (e < (int)seg_len) dst[e] = kraw[j];
        }
      }
      for (int e = tid; e < (int)seg_len; e += THREADS) {
        const unsigned int p = PACK ? (unsigned int)sw[smpad(e)] : (unsigned int)sp[smpad(e)];
        idst[e]              = (int64_t)p + index_offset;
      }
    }
    __syncthreads();  // all reads of shared memory are done before the next row's load
  }
}

}  // namespace b2s
