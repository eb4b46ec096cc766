// One-dimensional stable LSD radix sort for sm_100a: a single histogram sweep, then one
// "onesweep" pass per 8-bit digit with chained (decoupled look-back) tile prefixes.
// Stands in for cub::DeviceRadixSort::SortKeys / SortPairs as called by the reference
// (src/cupynumeric/sort/cub_sort.cuh:57-72,118-144); written from the published algorithm,
// it shares no code with CUB.
#pragma once

#include "b2s_common.cuh"

namespace b2s {

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
  uint32_t* idx_out32; // instead of idx_out: positions without offset, 32 bits wide
  const uint32_t* idx_in; // null: payloads are the element positions; else the caller's 32-bit payload
  void* tmp_keys[2];
  uint32_t* tmp_idx[2];
  unsigned int n;
  int npass;
  int key_bytes;
  uint4* zero_ptr;               // hist_kernel also clears this many 16-byte words (the look-back
  unsigned long long zero_vecs;  // tables of the passes) while it waits for its shared-memory atomics
};

// Body of the scan-and-route step, run by one whole CTA of at least RADIX threads (threads beyond
// the first RADIX only take part in the barriers).
__device__ __forceinline__ void scan_route_body(Ctrl* ctrl, const RouteArgs& a)
{
  __shared__ unsigned int warp_tot[RADIX / 32];
  __shared__ int active[MAX_PASSES];
  const int d    = threadIdx.x;
  const bool on  = d < RADIX;
  const int lane = d & 31, w = d >> 5;
  for (int p = 0; p < a.npass; ++p) {
    const unsigned int c = on ? ctrl->hist[p][d] : 0u;
    const int constant   = __syncthreads_or(on && c == a.n);
    unsigned int incl    = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (on && lane == 31) warp_tot[w] = incl;
    __syncthreads();
    if (on) {
      unsigned int base = 0;
      for (int i = 0; i < w; ++i) base += warp_tot[i];
      ctrl->hist[p][d] = base + incl - c;
    }
    if (d == 0) active[p] = !constant;
    __syncthreads();
  }
  if (d != 0) return;

  int m = 0;
  for (int p = 0; p < a.npass; ++p) m += active[p];
  const void* cur_keys   = a.keys_in;
  const uint32_t* cur_idx = a.idx_in;
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
        pd.dst_keys  = a.keys_out;
        pd.dst_idx64 = a.idx_out;
        pd.dst_idx32 = a.idx_out32;
        if (a.keys_out != nullptr && a.keys_out == cur_keys) {
          // a single effective pass over an in-place call: go through a temporary
          pd.dst_keys    = a.tmp_keys[0];
          fix.copy_src   = a.tmp_keys[0];
          fix.copy_dst   = a.keys_out;
          fix.copy_bytes = (unsigned long long)a.n * a.key_bytes;
        }
      } else {
        pd.dst_keys = a.tmp_keys[j & 1];
        pd.dst_idx32 = (a.idx_out || a.idx_out32) ? a.tmp_idx[j & 1] : nullptr;
      }
      cur_keys = pd.dst_keys;
      cur_idx  = pd.dst_idx32;
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
    fix.synth_idx   = a.idx_out;
    fix.synth_idx32 = a.idx_out32;
    fix.widen_src   = a.idx_in;
  }
  ctrl->fix = fix;
}

static __global__ void __launch_bounds__(RADIX) scan_route_kernel(Ctrl* ctrl, RouteArgs a) { scan_route_body(ctrl, a); }

// The digit histograms arrive ready-made in `nparts` pieces ([part][npass][RADIX] counts, e.g. one
// per rank that sent this GPU keys): add them up, then scan and route as usual.  Takes the place
// of the histogram kernel's read of all keys.
static __global__ void __launch_bounds__(RADIX)
hist_from_parts_kernel(Ctrl* ctrl, const unsigned int* __restrict__ parts, int nparts, RouteArgs a)
{
  const int d = threadIdx.x;
  for (int p = 0; p < a.npass; ++p) {
    unsigned int c = 0;
    for (int s = 0; s < nparts; ++s) c += parts[((size_t)s * a.npass + p) * RADIX + d];
    ctrl->hist[p][d] = c;
  }
  __syncthreads();
  scan_route_body(ctrl, a);
}

// ---------------------------------------------------------------------------------------------
// Kernel 1: digit histograms of every pass in one read of the keys: one shared-memory atomic per
// key and digit.  A warp-level shortcut for digits that all 32 lanes share (one lane adds 32;
// forms 0 and 1 below) was measured slower on every input, constant bytes and sorted keys
// included: 2^28 int64 keys with three constant bytes 0.91 -> 0.44 ms without it, nearly sorted
// uint64 0.96 -> 0.42, random float32 0.47 -> 0.40.  The hardware merges same-address atomics of a
// warp well enough, and the vote costs more than it saves.
// ---------------------------------------------------------------------------------------------
#ifndef B2S_HIST_FORM
#define B2S_HIST_FORM 2
#endif
template <int KB, int XF>
__device__ __forceinline__ void hist_add_full_warp(unsigned int (*sh)[RADIX], typename KeyOf<KB>::type raw)
{
  const auto k = to_ordered<KB, XF>(raw);
#pragma unroll
  for (int p = 0; p < KB; ++p) {
    const unsigned int d = (unsigned int)(k >> (8 * p)) & 0xFFu;
#if B2S_HIST_FORM == 1
    const int same = __all_sync(0xFFFFFFFFu, __shfl_sync(0xFFFFFFFFu, d, 0) == d);
#elif B2S_HIST_FORM == 2
    const int same = 0;
#else
    int same;
    __match_all_sync(0xFFFFFFFFu, d, &same);
#endif
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
hist_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned int n, Ctrl* ctrl, RouteArgs route)
{
  using K = typename KeyOf<KB>::type;
  __shared__ unsigned int sh[KB][RADIX];
  for (int i = threadIdx.x; i < KB * RADIX; i += HIST_THREADS) (&sh[0][0])[i] = 0;
  __syncthreads();

  // the look-back tables of the passes start out empty: cleared here, where the memory pipe is
  // mostly idle, instead of by a memset of their own in front of the sort
  for (unsigned long long i = (unsigned long long)blockIdx.x * HIST_THREADS + threadIdx.x; i < route.zero_vecs;
       i += (unsigned long long)gridDim.x * HIST_THREADS)
    route.zero_ptr[i] = make_uint4(0u, 0u, 0u, 0u);

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
  // The CTA that finishes last turns the complete histograms into digit bases and routes the
  // passes (what would otherwise be a launch of its own).
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&ctrl->hist_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  scan_route_body(ctrl, route);
}

// The same histograms with one copy of every table per lane (KB <= 4) or per pair of lanes
// (8-byte keys), laid out so that a lane's counters sit in the lane's own bank: an atomic
// instruction of a warp then costs one shared-memory wavefront (at most two for 8-byte keys) instead
// of the ~3 that 32 random digits cost in a single table - the single-table kernel is bound by
// exactly those bank conflicts.  One CTA of 1024 threads per SM holds the copies (128 KB).
constexpr int HISTL_THREADS = 1024;
template <int KB> struct HistLanes {
  static constexpr int COPIES   = KB <= 4 ? 32 : 16;
  static constexpr size_t BYTES = (size_t)KB * RADIX * COPIES * sizeof(unsigned int);
};

template <int KB, int XF>
__global__ void __launch_bounds__(HISTL_THREADS, 1)
hist_lanes_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned int n, Ctrl* ctrl, RouteArgs route)
{
  using K = typename KeyOf<KB>::type;
  constexpr int COPIES = HistLanes<KB>::COPIES;
  extern __shared__ __align__(16) unsigned int histl_smem[];
  unsigned int* sh = histl_smem;  // [(pass * RADIX + digit) * COPIES + copy]
  for (int i = threadIdx.x; i < KB * RADIX * COPIES; i += HISTL_THREADS) sh[i] = 0;
  for (unsigned long long i = (unsigned long long)blockIdx.x * HISTL_THREADS + threadIdx.x; i < route.zero_vecs;
       i += (unsigned long long)gridDim.x * HISTL_THREADS)
    route.zero_ptr[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();

  constexpr int VEC = 16 / KB;  // keys per 128-bit load
  constexpr int UNROLL = 4;     // loads in flight per thread
  const unsigned int copy    = threadIdx.x & (COPIES - 1);
  const bool aligned         = (reinterpret_cast<uintptr_t>(keys) & 15u) == 0;
  const unsigned int nvec    = aligned ? n / VEC : 0;
  const unsigned int gthread = blockIdx.x * HISTL_THREADS + threadIdx.x;
  const unsigned int gstride = gridDim.x * HISTL_THREADS;
  const uint4* vkeys         = reinterpret_cast<const uint4*>(keys);
  // Byte offset of a counter: table p starts at p * TABLE, a digit's copies at digit * ROW, mine at
  // copy * 4 (below ROW, so it can be OR-ed in): a shift, a logic operation and an add per digit,
  // then a reduction that returns nothing.
  constexpr unsigned int ROW = COPIES * 4, TABLE = RADIX * ROW;
  constexpr int ROW_LOG2     = COPIES == 32 ? 7 : 6;
  const unsigned int window  = (unsigned int)__cvta_generic_to_shared(sh);
  const unsigned int mine    = copy * 4u;
  auto add = [&](K raw) {
    const auto k = to_ordered<KB, XF>(raw);
#pragma unroll
    for (int p = 0; p < KB; ++p) {
      const int sh_by         = 8 * p - ROW_LOG2;  // digit << ROW_LOG2, taken straight from the key
      const unsigned int slot = (unsigned int)(sh_by >= 0 ? (k >> (sh_by >= 0 ? sh_by : 0)) : (k << (sh_by < 0 ? -sh_by : 0))) &
                                (0xFFu << ROW_LOG2);
      asm volatile("red.shared.add.u32 [%0], 1;" ::"r"((slot | mine) + (window + p * TABLE)) : "memory");
    }
  };
  unsigned int v = gthread;
  for (; v + (UNROLL - 1) * gstride < nvec; v += UNROLL * gstride) {
    uint4 q[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) q[u] = __ldg(vkeys + v + u * gstride);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      alignas(16) K tmp[VEC];
      *reinterpret_cast<uint4*>(tmp) = q[u];
#pragma unroll
      for (int j = 0; j < VEC; ++j) add(tmp[j]);
    }
  }
  for (; v < nvec; v += gstride) {
    alignas(16) K tmp[VEC];
    *reinterpret_cast<uint4*>(tmp) = __ldg(vkeys + v);
#pragma unroll
    for (int j = 0; j < VEC; ++j) add(tmp[j]);
  }
  for (unsigned int i = nvec * VEC + gthread; i < n; i += gstride) add(keys[i]);
  __syncthreads();
  // sum of the copies of every counter; thread t starts at copy t so that the threads of a warp
  // read different banks
  for (int i = threadIdx.x; i < KB * RADIX; i += HISTL_THREADS) {
    unsigned int c = 0;
#pragma unroll 8
    for (int j = 0; j < COPIES; ++j) c += sh[i * COPIES + ((j + threadIdx.x) & (COPIES - 1))];
    if (c) atomicAdd(&ctrl->hist[0][0] + i, c);
  }
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&ctrl->hist_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  scan_route_body(ctrl, route);
}

// ---------------------------------------------------------------------------------------------
// Per-segment variants of kernels 1 and 2 for segments too long for the on-chip sort: one CTA
// counts one chunk of one segment; a second kernel turns each 256-bin histogram into bases.
// ---------------------------------------------------------------------------------------------
constexpr unsigned int SEG_HIST_CHUNK = 8192;

template <int KB, int XF>
__global__ void __launch_bounds__(256)
seg_hist_kernel(const typename KeyOf<KB>::type* __restrict__ keys, unsigned int seg_len, unsigned int chunks_per_seg,
                unsigned int* __restrict__ seg_hist)
{
  __shared__ unsigned int sh[KB][RADIX];
  for (int i = threadIdx.x; i < KB * RADIX; i += 256) (&sh[0][0])[i] = 0;
  __syncthreads();
  const unsigned int seg = blockIdx.x / chunks_per_seg, chunk = blockIdx.x - seg * chunks_per_seg;
  const unsigned int lo  = chunk * SEG_HIST_CHUNK;
  const unsigned int hi  = min(seg_len, lo + SEG_HIST_CHUNK);
  const auto* base       = keys + (size_t)seg * seg_len;
  for (unsigned int i = lo + threadIdx.x; i < hi; i += 256) {
    const auto k = to_ordered<KB, XF>(base[i]);
#pragma unroll
    for (int p = 0; p < KB; ++p) atomicAdd(&sh[p][(unsigned int)(k >> (8 * p)) & 0xFFu], 1u);
  }
  __syncthreads();
  unsigned int* out = seg_hist + (size_t)seg * KB * RADIX;
  for (int i = threadIdx.x; i < KB * RADIX; i += 256) {
    const unsigned int c = (&sh[0][0])[i];
    if (c) atomicAdd(out + i, c);
  }
}

// One CTA of 256 threads per (segment, pass): counts -> exclusive bases, in place.
static __global__ void __launch_bounds__(RADIX) seg_scan_kernel(unsigned int* __restrict__ seg_hist)
{
  __shared__ unsigned int warp_tot[RADIX / 32];
  unsigned int* h      = seg_hist + (size_t)blockIdx.x * RADIX;
  const int d          = threadIdx.x, lane = d & 31, w = d >> 5;
  const unsigned int c = h[d];
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
  h[d] = base + incl - c;
}

// ---------------------------------------------------------------------------------------------
// Kernel 4: the rare leftovers described by FixDesc.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fixup_body(const FixDesc& f, unsigned int n, int64_t index_offset, size_t gthread, size_t gstride)
{
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
    if (f.widen_src != nullptr) {
      for (size_t i = gthread; i < n; i += gstride) f.synth_idx[i] = index_offset + (int64_t)f.widen_src[i];
    } else {
      for (size_t i = gthread; i < n; i += gstride) f.synth_idx[i] = index_offset + (int64_t)i;
    }
  }
  if (f.synth_idx32 != nullptr) {
    if (f.widen_src != nullptr) {
      for (size_t i = gthread; i < n; i += gstride) f.synth_idx32[i] = f.widen_src[i];
    } else {
      for (size_t i = gthread; i < n; i += gstride) f.synth_idx32[i] = (uint32_t)i;
    }
  }
}

// The rare leftovers: the copy of an in-place single-pass sort out of its temporary; keys that are
// all equal (no pass runs: copy, synthesised indices).  A launch of its own: as a call inside the
// radix pass it cost the keys-only passes 5 % (measured), far more than the launch.
static __global__ void __launch_bounds__(256) fixup_kernel(const Ctrl* ctrl, unsigned int n, int64_t index_offset)
{
  fixup_body(ctrl->fix, n, index_offset, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
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
//
// Ranking: a warp owns ITEMS*32 consecutive keys, element i of lane l at offset 32*i + l.  The
// ITEMS elements are split into CHAINS groups of consecutive elements; each group has its own
// row of 256 digit counters ("virtual warp"), so the CHAINS counter updates of one loop
// iteration are independent of each other and their shared-memory latencies overlap.
// ---------------------------------------------------------------------------------------------
#ifndef B2S_RANK_ATOMIC
#define B2S_RANK_ATOMIC 0
#endif
// 0: two lookups per key in the permutation; 1: digit starts folded into the row prefixes;
// 2: folded for key + index passes of keys up to 4 bytes only (measured: a gain there, a loss elsewhere)
#ifndef B2S_FOLD_EXCL
#define B2S_FOLD_EXCL 2
#endif
constexpr unsigned int LB_FLAG_AGG  = 1u << 30;  // tile count published
constexpr unsigned int LB_FLAG_INCL = 2u << 30;  // inclusive prefix published
constexpr unsigned int LB_VALUE     = (1u << 30) - 1;
constexpr unsigned int MAX_N_1D     = 1u << 30;  // counts must fit 30 bits
#ifndef B2S_CFG_LB_WINDOW
#define B2S_CFG_LB_WINDOW 4
#endif
constexpr int LB_WINDOW             = B2S_CFG_LB_WINDOW;  // predecessors inspected per round trip

template <int KB, bool PAIRS, int THREADS, int ITEMS, int CHAINS>
struct SweepSmem {
  static constexpr int TILE  = THREADS * ITEMS;
  static constexpr int WARPS = THREADS / 32;
  static constexpr int ROWS  = WARPS * CHAINS;  // counter rows ("virtual warps")
  static constexpr size_t KEY_BYTES = ((size_t)TILE * KB + 127) / 128 * 128;
  static constexpr size_t VAL_BYTES = PAIRS ? (size_t)TILE * 4 : 0;  // positions travel as 32 bits
  static constexpr size_t OFF_VALS  = KEY_BYTES;
  static constexpr size_t OFF_HIST  = OFF_VALS + VAL_BYTES;
  // B2S_RANK_ATOMIC: one 256-entry table of lane masks per warp, built with shared-memory atomicOr
  static constexpr size_t OFF_MASK  = OFF_HIST + (size_t)ROWS * RADIX * 4;
  static constexpr size_t OFF_EXCL  = OFF_MASK + (B2S_RANK_ATOMIC ? (size_t)WARPS * RADIX * 4 : 0);
  static constexpr size_t OFF_BASE  = OFF_EXCL + RADIX * 4;
  static constexpr size_t OFF_BAR   = OFF_BASE + RADIX * 4;
  static constexpr size_t OFF_MISC  = OFF_BAR + 8;
  static constexpr size_t BYTES     = OFF_MISC + 8;
};

// Segment geometry of a launch.  A 1-D sort is one segment of n keys.  Tiles never straddle
// segments: tile t belongs to segment t / tiles_per_seg, and each segment has its own chain of
// look-back entries (its first tile publishes an inclusive prefix at once) and its own digit
// bases (seg_bases; null for the 1-D case, whose bases live in the control block).
struct SegGeom {
  unsigned int seg_len;
  unsigned int tiles_per_seg;
  unsigned int nseg;
  int npass;
  const unsigned int* seg_bases;  // [nseg][npass][RADIX] exclusive digit bases, or null
};

template <int KB, int XF, bool PAIRS, int THREADS, int ITEMS, int CHAINS, int MIN_CTAS>
__global__ void __launch_bounds__(THREADS, MIN_CTAS)
onesweep_kernel(Ctrl* ctrl, unsigned int* __restrict__ lookback, int pass, SegGeom geo, int64_t index_offset)
{
  using K = typename KeyOf<KB>::type;
  using S = SweepSmem<KB, PAIRS, THREADS, ITEMS, CHAINS>;
  constexpr int TILE  = S::TILE;
  constexpr int ROWS  = S::ROWS;
  constexpr int IPC   = ITEMS / CHAINS;  // items per chain
  static_assert(THREADS >= RADIX, "one thread per digit is needed for the look-back");
  static_assert(ITEMS % CHAINS == 0, "chains split the items evenly");

  const PassDesc pd = ctrl->pass[pass];
  if (!pd.active) return;

  extern __shared__ __align__(128) unsigned char smem[];
  K* stage_keys          = reinterpret_cast<K*>(smem);
  uint32_t* stage_vals   = reinterpret_cast<uint32_t*>(smem + S::OFF_VALS);
  unsigned int* hist     = reinterpret_cast<unsigned int*>(smem + S::OFF_HIST);
  unsigned int* dig_excl = reinterpret_cast<unsigned int*>(smem + S::OFF_EXCL);
  unsigned int* base_ml  = reinterpret_cast<unsigned int*>(smem + S::OFF_BASE);
  uint64_t* bar          = reinterpret_cast<uint64_t*>(smem + S::OFF_BAR);
  unsigned int* misc     = reinterpret_cast<unsigned int*>(smem + S::OFF_MISC);

  const int tid  = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int shift   = pass * RADIX_BITS;
  const DigitSel ds = make_digit_sel<KB, XF>(pass);

  if (tid == 0) {
    // one thread reads the abort flag for the whole CTA, so that all of its threads leave together
    const unsigned int ticket = atomicAdd(&ctrl->tile_counter[pass], 1u);
    misc[1] = ld_relaxed(&ctrl->abort);
    misc[0] = ticket;
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  for (int i = tid; i < (ROWS + (B2S_RANK_ATOMIC ? S::WARPS : 0)) * RADIX; i += THREADS) hist[i] = 0;
  __syncthreads();
  if (misc[1]) return;
  const unsigned int tile = misc[0];
  const unsigned int seg  = tile / geo.tiles_per_seg;
  if (seg >= geo.nseg) return;  // more CTAs than tiles
  const unsigned int t_in      = tile - seg * geo.tiles_per_seg;  // tile number inside its segment
  const unsigned int tile_base = t_in * TILE;                     // first element, segment-relative
  const size_t seg_off         = (size_t)seg * geo.seg_len;
  const unsigned int valid     = min((unsigned int)TILE, geo.seg_len - tile_base);
  const K* src_keys            = static_cast<const K*>(pd.src_keys) + seg_off;
  const uint32_t* src_idx      = pd.src_idx ? pd.src_idx + seg_off : nullptr;
  const bool full          = valid == TILE;
  const bool load_idx      = PAIRS && src_idx != nullptr;
  const bool use_bulk      = full && ((reinterpret_cast<uintptr_t>(src_keys + tile_base) & 15u) == 0) &&
                        (!load_idx || (reinterpret_cast<uintptr_t>(src_idx + tile_base) & 15u) == 0);

  // ---- load the tile; keys end up in registers in warp-striped order ----
  K key[ITEMS];
  const int stripe0 = warp * (ITEMS * 32) + lane;  // element i of this thread sits at stripe0 + 32*i
  if (use_bulk) {
    int arrived = 1;
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)(TILE * KB) + (load_idx ? (uint32_t)(TILE * 4) : 0u);
      mbar_expect_tx(bar, bytes);
      bulk_load(stage_keys, src_keys + tile_base, TILE * KB, bar);
      if (load_idx) bulk_load(stage_vals, src_idx + tile_base, TILE * 4, bar);
      arrived = mbar_wait_bounded(bar, 0);  // one thread waits; the others park at the barrier
    }
    if (!__syncthreads_and(arrived)) {
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
        stage_vals[e]        = e < valid ? src_idx[tile_base + e] : 0;
      }
    }
  }

  // ---- stable in-warp ranking by digit: match lanes holding the same digit ----
  // rd[i] packs the element's digit (bits 16..23) with its rank among the same digit inside its
  // chain (bits 0..15).
  unsigned int rd[ITEMS];
  unsigned int* my_hist = hist + (warp * CHAINS) * RADIX;
  const unsigned int lt = lanemask_lt();
#if B2S_RANK_ATOMIC
  // Peer masks through shared memory: every lane ORs its bit into the mask of its digit, reads
  // the mask back, and the group clears it for the next element.  Far fewer instructions than
  // eight ballots, at the price of more shared-memory traffic.
  static_assert(CHAINS == 1, "the atomic form keeps one chain");
  unsigned int* my_mask       = hist + ROWS * RADIX + warp * RADIX;
  const unsigned int lane_bit = 1u << lane;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const unsigned int d = digit_fast<KB, XF>(key[k], ds, shift);
    atomicOr(&my_mask[d], lane_bit);
    __syncwarp();
    const unsigned int peers = my_mask[d];
    const unsigned int old   = my_hist[d];
    __syncwarp();
    my_hist[d] = old + __popc(peers);
    my_mask[d] = 0;
    __syncwarp();
    rd[k] = (d << 16) | (old + __popc(peers & lt));
  }
#else
#pragma unroll
  for (int k = 0; k < IPC; ++k) {
    unsigned int d[CHAINS], peers[CHAINS], old[CHAINS];
#pragma unroll
    for (int c = 0; c < CHAINS; ++c) {
      d[c]     = digit_fast<KB, XF>(key[c * IPC + k], ds, shift);
      peers[c] = warp_peers(d[c]);
    }
#pragma unroll
    for (int c = 0; c < CHAINS; ++c) old[c] = my_hist[c * RADIX + d[c]];
    __syncwarp();
#pragma unroll
    // every lane of a group stores the same value to the same counter: no leader election needed
    for (int c = 0; c < CHAINS; ++c) my_hist[c * RADIX + d[c]] = old[c] + __popc(peers[c]);
    __syncwarp();
#pragma unroll
    for (int c = 0; c < CHAINS; ++c) rd[c * IPC + k] = (d[c] << 16) | (old[c] + __popc(peers[c] & lt));
  }
#endif
  __syncthreads();

  // ---- per-digit tile counts: exclusive scan over the counter rows, then over the digits.  FOLD:
  // a second sweep over the rows adds the digit's start to every row's prefix, so that the
  // permutation below needs one table lookup per key instead of two (pays for the larger tiles of
  // the key + index passes; the keys-only tiles are too small to win it back) ----
  constexpr bool FOLD = B2S_FOLD_EXCL == 1 || (B2S_FOLD_EXCL == 2 && PAIRS && KB <= 4);
  unsigned int my_count = 0;
  if (tid < RADIX) {
    unsigned int run = 0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const unsigned int t  = hist[r * RADIX + tid];
      if (!FOLD) hist[r * RADIX + tid] = run;
      run += t;
    }
    my_count = run;
    unsigned int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) base_ml[warp] = incl;  // scratch: totals of the 8 digit groups
    dig_excl[tid] = incl - run;
  }
  __syncthreads();
  unsigned int my_excl_tile = 0;
  if (tid < RADIX) {
    unsigned int add = 0;
    for (int w = 0; w < warp; ++w) add += base_ml[w];
    my_excl_tile = dig_excl[tid] + add;
    if (FOLD) {
      unsigned int run = my_excl_tile;
#pragma unroll 1
      for (int r = 0; r < ROWS; ++r) {
        const unsigned int t  = hist[r * RADIX + tid];
        hist[r * RADIX + tid] = run;
        run += t;
      }
    }
  }
  __syncthreads();

  // ---- publish this tile's digit counts, then do local work before looking back ----
  // The permutation inside shared memory needs nothing from other tiles, so it runs between the
  // publication of the counts and the walk over the predecessors: by then most of them have
  // published too and the walk rarely has to poll.
  unsigned int* mine = lookback + (size_t)tile * RADIX + (tid < RADIX ? tid : 0);
  if (tid < RADIX) {
    if (!FOLD) dig_excl[tid] = my_excl_tile;
    st_relaxed(mine, (t_in == 0 ? LB_FLAG_INCL : LB_FLAG_AGG) | my_count);
  }
  if (!FOLD) __syncthreads();

  // ---- permute the tile inside shared memory: position = digit start + earlier rows + rank ----
  unsigned int pos[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const unsigned int d = rd[i] >> 16;
    pos[i]               = (FOLD ? 0u : dig_excl[d]) + my_hist[(i / IPC) * RADIX + d] + (rd[i] & 0xFFFFu);
    stage_keys[pos[i]]   = key[i];
  }
  if (PAIRS) {
    uint32_t val[ITEMS];
    if (load_idx) {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) val[i] = stage_vals[stripe0 + 32 * i];
    } else {
#pragma unroll
      for (int i = 0; i < ITEMS; ++i) val[i] = tile_base + stripe0 + 32 * i;
    }
    __syncthreads();  // every thread holds its indices before any slot is overwritten
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) stage_vals[pos[i]] = val[i];
  }

  // ---- chained prefix over tiles (decoupled look-back), one thread per digit ----
  if (tid < RADIX) {
    unsigned int excl = 0;
    if (t_in != 0) {
      // Walk back over the predecessors (the segment's first tile always holds an inclusive
      // prefix, so the walk never leaves the segment), LB_WINDOW of them per round trip: the loads of one
      // window are independent, so a run of tiles that have only published their counts costs
      // one memory latency per window instead of one per tile.
      int t              = (int)tile - 1;
      unsigned int spins = 0, spin_cap = SPIN_LIMIT;
      bool gave_up       = false;
      bool done          = false;
      while (!done) {
        unsigned int v[LB_WINDOW];
#pragma unroll
        for (int j = 0; j < LB_WINDOW; ++j) {
          const int tj = t - j;
          v[j]         = tj >= 0 ? ld_relaxed(lookback + (size_t)tj * RADIX + tid) : LB_FLAG_INCL;
        }
        int used = 0;
#pragma unroll
        for (int j = 0; j < LB_WINDOW; ++j) {
          if (!done && used == j) {
            const unsigned int f = v[j] >> 30;
            if (f != 0) {
              excl += v[j] & LB_VALUE;
              ++used;
              if (f == 2) done = true;
            }
          }
        }
        t -= used;
        if (!done && used == 0) {
          if (spins == 0 && ctrl->spin_limit != 0) spin_cap = ctrl->spin_limit;
          if (++spins > spin_cap || ((spins & 1023u) == 0 && ld_relaxed(&ctrl->abort))) {
            gave_up = true;
            break;
          }
          if (spins > 4) __nanosleep(64);  // leave the issue slots to the other CTAs of the SM
        }
      }
      if (gave_up) raise_timeout(ctrl);
      st_relaxed(mine, LB_FLAG_INCL | ((excl + my_count) & LB_VALUE));
    }
    // global index of a staged element = base_ml[digit] + its position in the staged tile
    const unsigned int* bases =
      geo.seg_bases ? geo.seg_bases + ((size_t)seg * geo.npass + pass) * RADIX : ctrl->hist[pass];
    base_ml[tid] = bases[tid] + excl - my_excl_tile;
  }
  __syncthreads();

  // ---- coalesced scatter: consecutive threads store consecutive elements of a digit's run ----
  K* dst_keys       = pd.dst_keys ? static_cast<K*>(pd.dst_keys) + seg_off : nullptr;
  uint32_t* dst_idx32 = pd.dst_idx32 ? pd.dst_idx32 + seg_off : nullptr;
  int64_t* dst_idx64  = pd.dst_idx64 ? pd.dst_idx64 + seg_off : nullptr;
  const bool wr_key = dst_keys != nullptr;
  if (full) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const unsigned int p = i * THREADS + tid;
      const K k            = stage_keys[p];
      const unsigned int g = base_ml[digit_fast<KB, XF>(k, ds, shift)] + p;
      if (wr_key) __stcg(dst_keys + g, k);
      if (PAIRS) {
        const uint32_t v = stage_vals[p];
        if (dst_idx64 != nullptr) __stcg(reinterpret_cast<long long*>(dst_idx64) + g, (long long)v + index_offset);
        else __stcg(dst_idx32 + g, v);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const unsigned int p = i * THREADS + tid;
      const K k            = stage_keys[p];
      const unsigned int g = base_ml[digit_fast<KB, XF>(k, ds, shift)] + p;
      if (p < valid) {
        if (wr_key) dst_keys[g] = k;
        if (PAIRS) {
          const uint32_t v = stage_vals[p];
          if (dst_idx64 != nullptr) dst_idx64[g] = (int64_t)v + index_offset;
          else dst_idx32[g] = v;
        }
      }
    }
  }
}

}  // namespace b2s
