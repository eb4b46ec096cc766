// Segmented sort for axis sorts: every segment (one row along the last axis) that fits in
// shared memory is loaded once, radix-sorted entirely on chip and stored once, so the HBM
// traffic is one read and one write per element whatever the key width.
// Stands in for cub::DeviceSegmentedRadixSort::SortKeys / SortPairs and for the short-segment
// thrust tuple sort (src/cupynumeric/sort/cub_sort.cuh:73-107,145-184,
// src/cupynumeric/sort/thrust_sort.cuh:61-123).
#pragma once

#include "b2s_common.cuh"

namespace b2s {

template <int KB, bool PAIRS, int THREADS, int ITEMS>
struct SegSmem {
  static constexpr int TILE           = THREADS * ITEMS;
  static constexpr int WARPS          = THREADS / 32;
  static constexpr size_t KEY_BYTES   = (size_t)TILE * KB;
  static constexpr size_t OFF_PAY     = (KEY_BYTES + 15) / 16 * 16;
  static constexpr size_t PAY_BYTES   = PAIRS ? (size_t)TILE * 4 : 0;
  static constexpr size_t OFF_WHIST   = OFF_PAY + PAY_BYTES;
  static constexpr size_t OFF_EXCL    = OFF_WHIST + (size_t)WARPS * RADIX * 4;
  static constexpr size_t OFF_RED     = OFF_EXCL + RADIX * 4;        // 2 x WARPS x 8 bytes
  static constexpr size_t OFF_BAR     = OFF_RED + (size_t)WARPS * 16;
  static constexpr size_t BYTES       = OFF_BAR + 16;
};

// One CTA sorts one segment at a time (grid-stride over segments). seg_len <= THREADS*ITEMS.
// PAIRS: the payload is the element's position inside its segment (32 bit on chip); the output
// index is payload + index_offset, which is both the 1-D rule (lo + i) and the N-D rule
// (i % L + lo_last) of src/cupynumeric/sort/sort.cu:1851-1862.
template <int KB, bool PAIRS, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS)
segsort_kernel(const typename KeyOf<KB>::type* __restrict__ in, typename KeyOf<KB>::type* __restrict__ out,
               int64_t* __restrict__ idx_out, unsigned int seg_len, unsigned long long nseg, int xf,
               int64_t index_offset, Ctrl* ctrl)
{
  using K = typename KeyOf<KB>::type;
  using S = SegSmem<KB, PAIRS, THREADS, ITEMS>;
  constexpr int TILE  = S::TILE;
  constexpr int WARPS = S::WARPS;

  extern __shared__ __align__(128) unsigned char smem[];
  K* skeys                = reinterpret_cast<K*>(smem);
  unsigned int* spay      = reinterpret_cast<unsigned int*>(smem + S::OFF_PAY);
  unsigned int* warp_hist = reinterpret_cast<unsigned int*>(smem + S::OFF_WHIST);
  unsigned int* dig_excl  = reinterpret_cast<unsigned int*>(smem + S::OFF_EXCL);
  unsigned long long* red = reinterpret_cast<unsigned long long*>(smem + S::OFF_RED);
  uint64_t* bar           = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);

  const int tid  = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int stripe0 = warp * (ITEMS * 32) + lane;
  const unsigned int lt = lanemask_lt();
  unsigned int* my_hist = warp_hist + warp * RADIX;
  const K pad           = pad_raw<KB>(xf);

  if (tid == 0) {
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  uint32_t phase = 0;

  const size_t seg_bytes = (size_t)seg_len * KB;
  for (unsigned long long seg = blockIdx.x; seg < nseg; seg += gridDim.x) {
    // one thread reads the abort flag; its answer reaches the others through the barrier below,
    // so the whole CTA leaves together
    int stop = 0;
    if (tid == 0) stop = (int)ld_relaxed(&ctrl->abort);
    const K* src = in + seg * seg_len;
    const bool use_bulk = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) && (seg_bytes % 16 == 0);
    if (use_bulk) {
      for (unsigned int e = seg_len + tid; e < TILE; e += THREADS) skeys[e] = pad;
      int arrived = 1;
      if (tid == 0 && !stop) {
        fence_proxy_async();  // earlier generic accesses to the buffer are ordered before the copy
        mbar_expect_tx(bar, (uint32_t)seg_bytes);
        bulk_load(skeys, src, (uint32_t)seg_bytes, bar);
        arrived = mbar_wait_bounded(bar, phase);  // one thread waits; the others park at the barrier
      }
      phase ^= 1u;
      if (!__syncthreads_and(arrived && !stop)) {
        if (tid == 0 && !stop) raise_timeout(ctrl);
        return;
      }
    } else {
      for (unsigned int e = tid; e < TILE; e += THREADS) skeys[e] = e < seg_len ? src[e] : pad;
      if (__syncthreads_or(stop)) return;
    }

    K key[ITEMS];
    unsigned int pay[PAIRS ? ITEMS : 1];
    // bits that differ between any two keys of the segment decide which passes matter
    K all_or = 0, all_and = (K)~(K)0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const unsigned int e = stripe0 + 32 * i;
      key[i]               = skeys[e];
      if (PAIRS) pay[i] = e;
      if (e < seg_len) {
        const K o = to_ordered_rt<KB>(key[i], xf);
        all_or |= o;
        all_and &= o;
      }
    }
    {
      unsigned long long o = all_or, a = all_and;
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) {
        o |= __shfl_xor_sync(0xFFFFFFFFu, o, s);
        a &= __shfl_xor_sync(0xFFFFFFFFu, a, s);
      }
      if (lane == 0) {
        red[2 * warp]     = o;
        red[2 * warp + 1] = a;
      }
      __syncthreads();
      o = 0;
      a = ~0ull;
      for (int w = 0; w < WARPS; ++w) {
        o |= red[2 * w];
        a &= red[2 * w + 1];
      }
      all_or  = (K)o;
      all_and = (K)a;
    }
    const K varying = (K)(all_or ^ all_and);

    for (int pass = 0; pass < KB; ++pass) {
      const int shift = pass * RADIX_BITS;
      if (((varying >> shift) & 0xFFu) == 0) continue;  // constant digit: identity pass
      for (int i = tid; i < WARPS * RADIX; i += THREADS) warp_hist[i] = 0;
      __syncthreads();
      unsigned int rank[ITEMS];
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const unsigned int d     = (unsigned int)(to_ordered_rt<KB>(key[i], xf) >> shift) & 0xFFu;
        const unsigned int peers = warp_peers(d);
        const unsigned int old   = my_hist[d];
        __syncwarp();
        my_hist[d] = old + __popc(peers);  // same value from every lane of the group
        __syncwarp();
        rank[i] = old + __popc(peers & lt);
      }
      __syncthreads();
      // exclusive scan over warps for each digit
      for (int d = tid; d < RADIX; d += THREADS) {
        unsigned int run = 0;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
          const unsigned int t     = warp_hist[w * RADIX + d];
          warp_hist[w * RADIX + d] = run;
          run += t;
        }
        dig_excl[d] = run;
      }
      __syncthreads();
      // exclusive scan over the 256 digit totals: warp 0, eight digits per lane
      if (warp == 0) {
        unsigned int c[8], sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          c[j] = dig_excl[lane * 8 + j];
          sum += c[j];
        }
        unsigned int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += t;
        }
        unsigned int run = incl - sum;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dig_excl[lane * 8 + j] = run;
          run += c[j];
        }
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const unsigned int d = (unsigned int)(to_ordered_rt<KB>(key[i], xf) >> shift) & 0xFFu;
        const unsigned int p = dig_excl[d] + my_hist[d] + rank[i];
        skeys[p]             = key[i];
        if (PAIRS) spay[p] = pay[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        key[i] = skeys[stripe0 + 32 * i];
        if (PAIRS) pay[i] = spay[stripe0 + 32 * i];
      }
      // the next pass (or the store below) only rewrites skeys after another barrier
    }

    // ---- store: the sorted segment sits in key[] / pay[] in striped order ----
    if (out != nullptr) {
      K* dst = out + seg * seg_len;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const unsigned int e = stripe0 + 32 * i;
        if (e < seg_len) dst[e] = key[i];
      }
    }
    if (PAIRS) {
      int64_t* dst = idx_out + seg * seg_len;
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const unsigned int e = stripe0 + 32 * i;
        if (e < seg_len) dst[e] = (int64_t)pay[i] + index_offset;
      }
    }
    __syncthreads();  // all reads of shared memory are done before the next segment's load
  }
}

}  // namespace b2s
