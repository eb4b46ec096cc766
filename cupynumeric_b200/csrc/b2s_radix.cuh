// One-dimensional stable LSD radix sort for sm_100a: a single histogram sweep, then one
// "onesweep" pass per 8-bit digit with chained (decoupled look-back) tile prefixes.
// Stands in for cub::DeviceRadixSort::SortKeys / SortPairs as called by the reference
// (src/cupynumeric/sort/cub_sort.cuh:57-72,118-144); written from the published algorithm,
// it shares no code with CUB.
#pragma once

#include "b2s_common.cuh"

namespace b2s {

// ---------------------------------------------------------------------------------------------
// Kernel 1: digit histograms of every pass in one read of the keys.
// Warp-level shortcut: when all 32 lanes hold the same digit (sorted input, constant high
// bytes) one lane adds 32 instead of 32 serialised shared-memory atomics.
// ---------------------------------------------------------------------------------------------
template <int KB, int XF>
__device__ __forceinline__ void hist_add_full_warp(unsigned int (*sh)[RADIX], typename KeyOf<KB>::type raw)
{
  const auto k = to_ordered<KB, XF>(raw);
#pragma unroll
  for (int p = 0; p < KB; ++p) {
    const unsigned int d = (unsigned int)(k >> (8 * p)) & 0xFFu;
    int same;
    __match_all_sync(0xFFFFFFFFu, d, &same);
    if (same) {
      if ((threadIdx.x & 31) == 0) atomicAdd(&sh[p][d], 32u);
    } else {
      atomicAdd(&sh[p][d], 1u);
    }
  }
}

constexpr int HIST_THREADS = 512;

template <int KB, int XF>
__global__ void __launch_bounds__(HIST_THREADS)
hist_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned int n, Ctrl* ctrl)
{
  using K = typename KeyOf<KB>::type;
  __shared__ unsigned int sh[KB][RADIX];
  for (int i = threadIdx.x; i < KB * RADIX; i += HIST_THREADS) (&sh[0][0])[i] = 0;
  __syncthreads();

  constexpr int VEC = 16 / KB;  // keys per 128-bit load
  const bool aligned = (reinterpret_cast<uintptr_t>(keys) & 15u) == 0;
  const unsigned int nvec = aligned ? n / VEC : 0;
  // Round the vector count down to whole warps so that the warp shortcut sees 32 live lanes.
  const unsigned int nvec_w  = nvec & ~31u;
  const unsigned int gthread = blockIdx.x * HIST_THREADS + threadIdx.x;
  const unsigned int gstride = gridDim.x * HIST_THREADS;
  const uint4* vkeys         = reinterpret_cast<const uint4*>(keys);
  for (unsigned int v = gthread; v < nvec_w; v += gstride) {
    const uint4 q = __ldg(vkeys + v);
    alignas(16) K tmp[VEC];
    *reinterpret_cast<uint4*>(tmp) = q;
#pragma unroll
    for (int j = 0; j < VEC; ++j) hist_add_full_warp<KB, XF>(sh, tmp[j]);
  }
  // remainder: plain atomics
  for (unsigned int i = nvec_w * VEC + gthread; i < n; i += gstride) {
    const auto k = to_ordered<KB, XF>(keys[i]);
#pragma unroll
    for (int p = 0; p < KB; ++p) atomicAdd(&sh[p][(unsigned int)(k >> (8 * p)) & 0xFFu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < KB * RADIX; i += HIST_THREADS) {
    const unsigned int c = (&sh[0][0])[i];
    if (c) atomicAdd(&ctrl->hist[0][0] + i, c);
  }
}

// ---------------------------------------------------------------------------------------------
// Kernel 2 (one CTA): turn the histograms into exclusive digit bases, find passes whose digit is
// constant over the array (a stable pass over a constant digit is the identity, so it is
// skipped) and route the remaining passes through the two temporaries so that the last one
// lands in the caller's output.
// ---------------------------------------------------------------------------------------------
struct RouteArgs {
  const void* keys_in;
  void* keys_out;     // may be null (argsort)
  int64_t* idx_out;   // may be null (sort)
  void* tmp_keys[2];
  int64_t* tmp_idx[2];
  unsigned int n;
  int npass;
  int key_bytes;
};

static __global__ void __launch_bounds__(RADIX) scan_route_kernel(Ctrl* ctrl, RouteArgs a)
{
  __shared__ unsigned int warp_tot[RADIX / 32];
  __shared__ int active[MAX_PASSES];
  const int d    = threadIdx.x;
  const int lane = d & 31, w = d >> 5;
  for (int p = 0; p < a.npass; ++p) {
    const unsigned int c = ctrl->hist[p][d];
    const int constant   = __syncthreads_or(c == a.n);
    unsigned int incl    = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[w] = incl;
    __syncthreads();
    unsigned int base = 0;
    for (int i = 0; i < w; ++i) base += warp_tot[i];
    ctrl->hist[p][d] = base + incl - c;
    if (d == 0) active[p] = !constant;
    __syncthreads();
  }
  if (d != 0) return;

  int m = 0;
  for (int p = 0; p < a.npass; ++p) m += active[p];
  const void* cur_keys   = a.keys_in;
  const int64_t* cur_idx = nullptr;
  FixDesc fix            = {};
  int j                  = 0;
  for (int p = 0; p < a.npass; ++p) {
    PassDesc pd = {};
    pd.active   = active[p];
    if (active[p]) {
      const bool last = (j == m - 1);
      pd.src_keys     = cur_keys;
      pd.src_idx      = cur_idx;
      if (last) {
        pd.dst_keys = a.keys_out;
        pd.dst_idx  = a.idx_out;
        if (a.keys_out != nullptr && a.keys_out == cur_keys) {
          // a single effective pass over an in-place call: go through a temporary
          pd.dst_keys    = a.tmp_keys[0];
          fix.copy_src   = a.tmp_keys[0];
          fix.copy_dst   = a.keys_out;
          fix.copy_bytes = (unsigned long long)a.n * a.key_bytes;
        }
      } else {
        pd.dst_keys = a.tmp_keys[j & 1];
        pd.dst_idx  = a.idx_out ? a.tmp_idx[j & 1] : nullptr;
      }
      cur_keys = pd.dst_keys;
      cur_idx  = pd.dst_idx;
      ++j;
    }
    ctrl->pass[p] = pd;
  }
  if (m == 0) {
    // already sorted as far as a radix sort can tell: every key is the same
    if (a.keys_out != nullptr && a.keys_out != a.keys_in) {
      fix.copy_src   = a.keys_in;
      fix.copy_dst   = a.keys_out;
      fix.copy_bytes = (unsigned long long)a.n * a.key_bytes;
    }
    fix.synth_idx = a.idx_out;
  }
  ctrl->fix = fix;
}

// ---------------------------------------------------------------------------------------------
// Kernel 4: the rare leftovers described by FixDesc.
// ---------------------------------------------------------------------------------------------
static __global__ void __launch_bounds__(256) fixup_kernel(const Ctrl* ctrl, unsigned int n, int64_t index_offset)
{
  const FixDesc f         = ctrl->fix;
  const size_t gthread    = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gstride    = (size_t)gridDim.x * blockDim.x;
  if (f.copy_src != nullptr) {
    const unsigned char* s = static_cast<const unsigned char*>(f.copy_src);
    unsigned char* d       = static_cast<unsigned char*>(f.copy_dst);
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15u) == 0) {
      const size_t nv = f.copy_bytes / 16;
      for (size_t i = gthread; i < nv; i += gstride)
        reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
      for (size_t i = nv * 16 + gthread; i < f.copy_bytes; i += gstride) d[i] = s[i];
    } else {
      for (size_t i = gthread; i < f.copy_bytes; i += gstride) d[i] = s[i];
    }
  }
  if (f.synth_idx != nullptr) {
    for (size_t i = gthread; i < n; i += gstride) f.synth_idx[i] = index_offset + (int64_t)i;
  }
}

// ---------------------------------------------------------------------------------------------
// Kernel 3: one onesweep pass.  A CTA takes the next tile (ticket from an atomic counter, so
// every predecessor of a tile is already running or done), ranks its keys stably by the pass's
// digit with warp-level match ranking, chains the per-digit tile counts to its predecessors
// through a look-back table (flag and count share one 32-bit word), and scatters the tile
// through shared memory so that each digit's run leaves as contiguous, coalesced stores.
//
// Key tiles (and index tiles) arrive by bulk asynchronous copy (TMA engine) when source and
// size are 16-byte multiples; the last, partial tile and unaligned sources use plain loads.
// ---------------------------------------------------------------------------------------------
constexpr unsigned int LB_FLAG_AGG  = 1u << 30;  // tile count published
constexpr unsigned int LB_FLAG_INCL = 2u << 30;  // inclusive prefix published
constexpr unsigned int LB_VALUE     = (1u << 30) - 1;
constexpr unsigned int MAX_N_1D     = 1u << 30;  // counts must fit 30 bits

template <int KB, bool PAIRS, int THREADS, int ITEMS>
struct SweepSmem {
  static constexpr int TILE  = THREADS * ITEMS;
  static constexpr int WARPS = THREADS / 32;
  // staging buffer: key tile, reused for the sorted keys, then (pairs) for the sorted indices
  static constexpr size_t STAGE_BYTES = (size_t)TILE * (PAIRS ? 8 : KB);
  static constexpr size_t VAL_BYTES   = PAIRS ? (size_t)TILE * 8 : 0;  // index tile as loaded
  static constexpr size_t OFF_VALS    = STAGE_BYTES;
  static constexpr size_t OFF_WHIST   = OFF_VALS + VAL_BYTES;
  static constexpr size_t OFF_EXCL    = OFF_WHIST + (size_t)WARPS * RADIX * 4;
  static constexpr size_t OFF_BASE    = OFF_EXCL + RADIX * 4;
  static constexpr size_t OFF_BAR     = OFF_BASE + RADIX * 4;
  static constexpr size_t OFF_MISC    = OFF_BAR + 8;
  static constexpr size_t BYTES       = OFF_MISC + 8;
};

template <int KB, int XF, bool PAIRS, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS)
onesweep_kernel(Ctrl* ctrl, unsigned int* __restrict__ lookback, int pass, unsigned int n, int64_t index_offset)
{
  using K = typename KeyOf<KB>::type;
  using S = SweepSmem<KB, PAIRS, THREADS, ITEMS>;
  constexpr int TILE  = S::TILE;
  constexpr int WARPS = S::WARPS;
  static_assert(THREADS >= RADIX, "one thread per digit is needed for the look-back");

  const PassDesc pd = ctrl->pass[pass];
  if (!pd.active) return;
  if (ld_relaxed(&ctrl->abort)) return;

  extern __shared__ __align__(128) unsigned char smem[];
  K* stage_keys           = reinterpret_cast<K*>(smem);
  int64_t* stage_vals     = reinterpret_cast<int64_t*>(smem);
  int64_t* in_vals        = reinterpret_cast<int64_t*>(smem + S::OFF_VALS);
  unsigned int* warp_hist = reinterpret_cast<unsigned int*>(smem + S::OFF_WHIST);
  unsigned int* dig_excl  = reinterpret_cast<unsigned int*>(smem + S::OFF_EXCL);
  unsigned int* base_ml   = reinterpret_cast<unsigned int*>(smem + S::OFF_BASE);
  uint64_t* bar           = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  unsigned int* misc      = reinterpret_cast<unsigned int*>(smem + S::OFF_MISC);

  const int tid  = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int shift = pass * RADIX_BITS;

  const K* src_keys      = static_cast<const K*>(pd.src_keys);
  const int64_t* src_idx = pd.src_idx;

  if (tid == 0) {
    misc[0] = atomicAdd(&ctrl->tile_counter[pass], 1u);
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  for (int i = tid; i < WARPS * RADIX; i += THREADS) warp_hist[i] = 0;
  __syncthreads();
  const unsigned int tile      = misc[0];
  const unsigned int tile_base = tile * TILE;
  if (tile_base >= n) return;  // more CTAs than tiles
  const unsigned int valid = min((unsigned int)TILE, n - tile_base);
  const bool full          = valid == TILE;
  const bool load_idx      = PAIRS && src_idx != nullptr;
  const bool use_bulk      = full && ((reinterpret_cast<uintptr_t>(src_keys) & 15u) == 0) &&
                        (!load_idx || (reinterpret_cast<uintptr_t>(src_idx) & 15u) == 0);

  // ---- load the tile; keys end up in registers in warp-striped order ----
  K key[ITEMS];
  const int stripe0 = warp * (ITEMS * 32) + lane;  // element i of this thread sits at stripe0 + 32*i
  if (use_bulk) {
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(TILE * KB) + (load_idx ? (uint32_t)(TILE * 8) : 0u);
      mbar_expect_tx(bar, bytes);
      bulk_load(stage_keys, src_keys + tile_base, TILE * KB, bar);
      if (load_idx) bulk_load(in_vals, src_idx + tile_base, TILE * 8, bar);
    }
    if (!mbar_wait_bounded(bar, 0)) {
      // The copy never signalled: record it and leave. Nothing was published for this tile, so
      // later tiles see `abort` in their own look-back loop and leave as well.
      if (tid == 0) raise_timeout(ctrl);
      return;
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) key[i] = stage_keys[stripe0 + 32 * i];
  } else {
    const K pad = pad_raw<KB>(XF);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const unsigned int e = stripe0 + 32 * i;
      key[i]               = e < valid ? src_keys[tile_base + e] : pad;
    }
    if (load_idx) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) {
        const unsigned int e = stripe0 + 32 * i;
        in_vals[e]           = e < valid ? src_idx[tile_base + e] : 0;
      }
    }
  }

  // ---- stable in-warp ranking by digit: match lanes holding the same digit ----
  unsigned int rank[ITEMS];
  unsigned int* my_hist = warp_hist + warp * RADIX;
  const unsigned int lt = lanemask_lt();
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const unsigned int d     = digit_of<KB, XF>(key[i], shift);
    const unsigned int peers = __match_any_sync(0xFFFFFFFFu, d);
    const unsigned int below = peers & lt;
    unsigned int old         = 0;
    if (below == 0) {  // lowest lane of the group owns the counter update
      old        = my_hist[d];
      my_hist[d] = old + __popc(peers);
    }
    __syncwarp();
    old     = __shfl_sync(0xFFFFFFFFu, old, __ffs(peers) - 1);
    rank[i] = old + __popc(below);
  }
  __syncthreads();

  // ---- per-digit tile counts: exclusive scan over warps, then over digits ----
  unsigned int my_count = 0;
  if (tid < RADIX) {
    unsigned int run = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const unsigned int t       = warp_hist[w * RADIX + tid];
      warp_hist[w * RADIX + tid] = run;
      run += t;
    }
    my_count = run;
    // exclusive scan of the 256 counts
    unsigned int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) base_ml[warp] = incl;  // scratch: warp totals (8 of them)
    dig_excl[tid] = incl - run;
  }
  __syncthreads();
  unsigned int my_excl_tile = 0;
  if (tid < RADIX) {
    unsigned int add = 0;
    for (int w = 0; w < warp; ++w) add += base_ml[w];
    my_excl_tile = dig_excl[tid] + add;
  }
  __syncthreads();

  // ---- chained prefix over tiles (decoupled look-back), one thread per digit ----
  if (tid < RADIX) {
    dig_excl[tid]       = my_excl_tile;
    unsigned int* mine  = lookback + (size_t)tile * RADIX + tid;
    unsigned int excl   = 0;
    if (tile == 0) {
      st_relaxed(mine, LB_FLAG_INCL | my_count);
    } else {
      st_relaxed(mine, LB_FLAG_AGG | my_count);
      unsigned int t     = tile - 1;
      unsigned int spins = 0;
      bool gave_up       = false;
      while (true) {
        const unsigned int v = ld_relaxed(lookback + (size_t)t * RADIX + tid);
        const unsigned int f = v >> 30;
        if (f == 0) {
          if (++spins > SPIN_LIMIT || ((spins & 1023u) == 0 && ld_relaxed(&ctrl->abort))) {
            gave_up = true;
            break;
          }
          continue;
        }
        excl += v & LB_VALUE;
        if (f == 2 || t == 0) break;
        --t;
      }
      if (gave_up) raise_timeout(ctrl);
      st_relaxed(mine, LB_FLAG_INCL | ((excl + my_count) & LB_VALUE));
    }
    // global index of a staged element = base_ml[digit] + its position in the staged tile
    base_ml[tid] = ctrl->hist[pass][tid] + excl - my_excl_tile;
  }
  __syncthreads();

  // ---- scatter keys through shared memory ----
  unsigned int pos[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const unsigned int d = digit_of<KB, XF>(key[i], shift);
    pos[i]               = dig_excl[d] + my_hist[d] + rank[i];
    stage_keys[pos[i]]   = key[i];
  }
  __syncthreads();
  K* dst_keys = static_cast<K*>(pd.dst_keys);
  unsigned int gidx[PAIRS ? ITEMS : 1];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const unsigned int p = i * THREADS + tid;
    const K k            = stage_keys[p];
    const unsigned int g = base_ml[digit_of<KB, XF>(k, shift)] + p;
    if (PAIRS) gidx[i] = g;
    if (dst_keys != nullptr && p < valid) dst_keys[g] = k;
  }

  // ---- indices follow the same permutation ----
  if (PAIRS) {
    int64_t val[ITEMS];
    if (load_idx) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) val[i] = in_vals[stripe0 + 32 * i];
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) val[i] = index_offset + (int64_t)(tile_base + stripe0 + 32 * i);
    }
    __syncthreads();  // every thread is done reading the staged keys
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) stage_vals[pos[i]] = val[i];
    __syncthreads();
    int64_t* dst_idx = pd.dst_idx;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const unsigned int p = i * THREADS + tid;
      if (p < valid) dst_idx[gidx[i]] = stage_vals[p];
    }
  }
}

}  // namespace b2s
