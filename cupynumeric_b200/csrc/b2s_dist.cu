// Distributed 1-D sort over the GPUs of one NVSwitch box, as a partition-first sample sort:
//   samples of the unsorted tile -> all-gather -> weighted splitters (on the device) ->
//   every element is classified by (key, rank, position) and written straight into the receive
//   buffer of its destination GPU by the partition kernel (plain stores over NVLink) ->
//   one barrier -> each GPU sorts what it received with the local radix sort.
// The runs a GPU receives lie in source-rank order and keep their input order, so the stable
// local sort of their concatenation is the global stable sort; no merge is needed.
// Replaces sample_sort_nccl_nd for 1-D arrays (src/cupynumeric/sort/sort.cu:1270-1784), which
// sorts first, exchanges through NCCL and merges in log2(P) sweeps, and the surrounding buffer
// handling of SortImplBody<GPU> (sort.cu:1797-1940).
//
// Also here: the stable k-way merge entry point (used by local sorts of 2^30 keys and more) and
// the move of variable-length parts into fixed extents (rebalance).
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_peer.cuh"

namespace b2s {
// defined with the local sort
bool local_sort_pos32_supported(size_t n);
int local_sort_payload32(int dtype, const void* keys_in, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                         int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, int out32 = 0);
int local_sort_received(int dtype, const void* keys_in, void* keys_out, const uint32_t* pay_in, int64_t* idx_out, size_t n,
                        int64_t index_offset, void* ws, size_t ws_bytes, cudaStream_t stream, const unsigned int* hist_parts,
                        int nparts);
}  // namespace b2s
#include "b2s_dist_host.h"
#include "b2s_merge.cuh"
#include "b2s_partition.cuh"
#include "b2s_prof.h"

namespace b2s {

static int kb_of(int dtype, int* xf)
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
    case B2S_COMPLEX128: *xf = XF_CFLOAT; return 16;  // (real, imaginary) doubles: a two-word key
    default: return 0;
  }
}

// ---------------------------------------------------------------------------------------------
// Keys as the partition kernels see them: raw storage type and two-word ordered image.
// ---------------------------------------------------------------------------------------------
template <int KB> struct DKey {
  using Raw = typename KeyOf<KB>::type;
  static __device__ __forceinline__ OKey okey(Raw r, int xf) { return OKey{(unsigned long long)to_ordered_rt<KB>(r, xf), 0ull}; }
};
template <> struct DKey<16> {
  using Raw = ulonglong2;  // x: bits of the real part, y: bits of the imaginary part
  static __device__ __forceinline__ OKey okey(Raw r, int)
  {
    return OKey{to_ordered<8, XF_FLOAT>(r.x), to_ordered<8, XF_FLOAT>(r.y)};
  }
};

// What every rank contributes to the first all-gather.
struct BlockA {
  long long n_local;
  long long global_offset;
  long long status;        // a b2s_status_t: this rank's failure so far
  long long capacity;      // elements its receive buffers hold
  long long reserved[4];
  PeerRecord rec;          // where the others can write (receive keys, receive payload)
  OKey okey[SAMPLES_PER_RANK];
};

// ... and to the second one.
struct BlockB {
  long long status;
  long long mapped;                 // 1: this rank can write into every rank's receive buffers
  long long total[MAX_BUCKETS];     // elements of my tile per destination
  long long reserved[6];
};

// Regular samples of the unsorted tile: ordered keys only; rank, position and weight follow
// from the slot number and the tile size (sample_position / sample_weight).
template <int KB>
__global__ void sample_kernel(const typename DKey<KB>::Raw* __restrict__ keys, long long n, int xf, OKey* __restrict__ out)
{
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= SAMPLES_PER_RANK) return;
  const long long s_eff = n < SAMPLES_PER_RANK ? n : SAMPLES_PER_RANK;
  out[j] = j < s_eff ? DKey<KB>::okey(keys[sample_position(j, s_eff, n)], xf) : OKey{~0ull, ~0ull};
}

// Gathered blocks -> one Sample per slot (rank-major, positions ascending inside a rank, which
// is the triple order among equal keys) and the two words the samples are ordered by.
__global__ void build_samples_kernel(const BlockA* __restrict__ blocks, int nranks, Sample* __restrict__ samples,
                                     unsigned long long* __restrict__ key_hi, unsigned long long* __restrict__ key_lo)
{
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= nranks * SAMPLES_PER_RANK) return;
  const int r = t / SAMPLES_PER_RANK, j = t % SAMPLES_PER_RANK;
  const long long n = blocks[r].n_local;
  const long long s_eff = n < SAMPLES_PER_RANK ? n : SAMPLES_PER_RANK;
  Sample s;
  s.rank = r;
  s.pad_ = 0;
  if (j < s_eff) {
    s.okey   = blocks[r].okey[j];
    s.pos    = sample_position(j, s_eff, n);
    s.weight = sample_weight(j, s_eff, n);
  } else {
    s.okey   = OKey{~0ull, ~0ull};
    s.pos    = 0;
    s.weight = 0;
  }
  samples[t] = s;
  key_hi[t]  = s.okey.hi;
  key_lo[t]  = s.okey.lo;
}

// out[i] = in[order[i]]
__global__ void gather_u64_kernel(const unsigned long long* __restrict__ in, const int64_t* __restrict__ order, int n,
                                  unsigned long long* __restrict__ out)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[order[i]];
}
// out[i] = first[second[i]]
__global__ void compose_kernel(const int64_t* __restrict__ first, const int64_t* __restrict__ second, int n, int64_t* __restrict__ out)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = first[second[i]];
}

// One CTA: cumulative weights along the ordered samples, then splitter k = the first sample whose
// inclusive cumulative weight reaches splitter_target(k); written in global form (all ranks get
// the same) and localised for `my_rank`.  `cum` is scratch for `count` values.
constexpr int SELECT_THREADS = 1024;
__global__ void __launch_bounds__(SELECT_THREADS)
select_splitters_kernel(const Sample* __restrict__ samples, const int64_t* __restrict__ order, int count, int nb, int my_rank,
                        long long* __restrict__ cum, Sample* __restrict__ splitters, LocalSplitter* __restrict__ local, int nlocal)
{
  __shared__ long long part[SELECT_THREADS];
  const int tid = threadIdx.x;
  const int per = (count + SELECT_THREADS - 1) / SELECT_THREADS;
  const int lo = min(tid * per, count), hi = min(lo + per, count);
  long long sum = 0;
  for (int t = lo; t < hi; ++t) sum += samples[order[t]].weight;
  part[tid] = sum;
  __syncthreads();
  for (int o = 1; o < SELECT_THREADS; o <<= 1) {
    const long long v = tid >= o ? part[tid - o] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  long long run = part[tid] - sum;
  for (int t = lo; t < hi; ++t) {
    run += samples[order[t]].weight;
    cum[t] = run;
  }
  const long long total = part[SELECT_THREADS - 1];
  __syncthreads();  // cum[] was written by this CTA only: visible to all of its threads now
  if (tid < nlocal) {
    Sample sp{};
    sp.okey = OKey{~0ull, ~0ull};
    if (tid < nb - 1 && total > 0) {
      const long long target = splitter_target(tid + 1, total, nb);
      int a = 0, b = count;  // first t with cum[t] >= target
      while (a < b) {
        const int m = (a + b) >> 1;
        if (cum[m] < target) a = m + 1; else b = m;
      }
      if (a < count) sp = samples[order[a]];
    }
    if (tid < nb - 1) splitters[tid] = sp;
    local[tid] = localise(sp, my_rank);
  }
}

// ---------------------------------------------------------------------------------------------
// The partition of a tile: a counting pass, a scan over tiles, a scatter pass.
// ---------------------------------------------------------------------------------------------
constexpr int PART_THREADS = 256;
constexpr int PART_ITEMS   = 16;
constexpr int PART_TILE    = PART_THREADS * PART_ITEMS;
constexpr int PART_WARPS   = PART_THREADS / 32;
constexpr unsigned int NO_BUCKET = 0xFFu;

// Destination of an element of the tile; `nsplit` = padded bucket count - 1 (padding splitters
// are invalid, nothing lies right of them), so the search takes the same steps for every lane.
__device__ __forceinline__ unsigned int classify(const LocalSplitter* split, int nsplit, const OKey& k, long long pos)
{
  return (unsigned int)bucket_of(split, nsplit, k, pos);
}

template <int KB>
__global__ void __launch_bounds__(PART_THREADS)
part_count_kernel(const typename DKey<KB>::Raw* __restrict__ keys, long long n, int xf, const LocalSplitter* __restrict__ split,
                  int nbp, unsigned int* __restrict__ tile_counts)
{
  __shared__ LocalSplitter ssplit[MAX_BUCKETS];
  __shared__ unsigned int cnt[MAX_BUCKETS];
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < nbp - 1) ssplit[tid] = split[tid];
  if (tid < MAX_BUCKETS) cnt[tid] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * PART_TILE;
  // all loads of the thread are issued before the first use, so that their latencies overlap
  typename DKey<KB>::Raw key[PART_ITEMS];
#pragma unroll
  for (int i = 0; i < PART_ITEMS; ++i) {
    const long long e = base + (long long)i * PART_THREADS + tid;
    if (e < n) key[i] = keys[e];
  }
#pragma unroll
  for (int i = 0; i < PART_ITEMS; ++i) {
    const long long e = base + (long long)i * PART_THREADS + tid;
    unsigned int b    = NO_BUCKET;
    if (e < n) b = classify(ssplit, nbp - 1, DKey<KB>::okey(key[i], xf), e);
    const unsigned int peers = __match_any_sync(0xFFFFFFFFu, b);
    if (b != NO_BUCKET && lane == __ffs(peers) - 1) atomicAdd(&cnt[b], (unsigned int)__popc(peers));
  }
  __syncthreads();
  if (tid < nbp) tile_counts[(size_t)blockIdx.x * nbp + tid] = cnt[tid];
}

// Bucket b = blockIdx.x: exclusive prefix of its per-tile counts over the tiles, and its total.
constexpr int SCAN_THREADS = 1024;
__global__ void __launch_bounds__(SCAN_THREADS)
tile_scan_kernel(const unsigned int* __restrict__ tile_counts, long long ntiles, int nbp, unsigned long long* __restrict__ tile_off,
                 long long* __restrict__ totals)
{
  __shared__ unsigned long long part[SCAN_THREADS];
  const int b = blockIdx.x, tid = threadIdx.x;
  const long long per = (ntiles + SCAN_THREADS - 1) / SCAN_THREADS;
  const long long lo = min((long long)tid * per, ntiles), hi = min(lo + per, ntiles);
  unsigned long long sum = 0;
  for (long long t = lo; t < hi; ++t) sum += tile_counts[t * nbp + b];
  part[tid] = sum;
  __syncthreads();
  for (int o = 1; o < SCAN_THREADS; o <<= 1) {
    const unsigned long long v = tid >= o ? part[tid - o] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  unsigned long long run = part[tid] - sum;
  for (long long t = lo; t < hi; ++t) {
    tile_off[t * nbp + b] = run;
    run += tile_counts[t * nbp + b];
  }
  if (tid == SCAN_THREADS - 1) totals[b] = (long long)part[tid];
}

// Where the elements of each bucket go: the destination rank's receive buffers, already advanced
// to the start of this rank's run in them.
struct PartDst {
  void* keys[MAX_BUCKETS];
  void* pay[MAX_BUCKETS];
};

template <int KB, int PAYB> struct PartSmem {
  static constexpr size_t KEY_BYTES = (size_t)PART_TILE * KB;
  static constexpr size_t OFF_PAY   = KEY_BYTES;
  static constexpr size_t OFF_SPLIT = OFF_PAY + (size_t)PART_TILE * PAYB;
  static constexpr size_t OFF_WCNT  = OFF_SPLIT + sizeof(LocalSplitter) * MAX_BUCKETS;
  static constexpr size_t OFF_START = OFF_WCNT + (size_t)PART_WARPS * MAX_BUCKETS * 4;  // MAX_BUCKETS + 1 entries
  static constexpr size_t OFF_GOFF  = (OFF_START + (MAX_BUCKETS + 1) * 4 + 7) / 8 * 8;
  static constexpr size_t OFF_DKEY  = OFF_GOFF + MAX_BUCKETS * 8;
  static constexpr size_t OFF_DPAY  = OFF_DKEY + MAX_BUCKETS * 8;
  static constexpr size_t BYTES     = OFF_DPAY + MAX_BUCKETS * 8;
};

// Stable partition of one tile: every element gets its rank among the tile's elements of the
// same bucket (in input order), the tile is staged bucket by bucket in shared memory, and each
// bucket's piece leaves as one contiguous, coalesced run - into this GPU's memory or, through a
// peer mapping, another GPU's.  PAYB: 0 no payload, 4 the element's global position minus
// `pay_base` as 32 bits, 8 its global position as int64.
template <int KB, int PAYB>
__global__ void __launch_bounds__(PART_THREADS)
part_scatter_kernel(const typename DKey<KB>::Raw* __restrict__ keys, long long n, int xf, const LocalSplitter* __restrict__ split,
                    int nbp, const unsigned long long* __restrict__ tile_off, const __grid_constant__ PartDst dst,
                    long long global_offset, long long pay_base)
{
  using Raw = typename DKey<KB>::Raw;
  using S   = PartSmem<KB, PAYB>;
  extern __shared__ __align__(16) unsigned char smem[];
  Raw* skeys                  = reinterpret_cast<Raw*>(smem);
  unsigned char* spay         = smem + S::OFF_PAY;
  LocalSplitter* ssplit       = reinterpret_cast<LocalSplitter*>(smem + S::OFF_SPLIT);
  unsigned int* wcnt          = reinterpret_cast<unsigned int*>(smem + S::OFF_WCNT);
  unsigned int* bstart        = reinterpret_cast<unsigned int*>(smem + S::OFF_START);
  unsigned long long* goff    = reinterpret_cast<unsigned long long*>(smem + S::OFF_GOFF);
  void** dkey                 = reinterpret_cast<void**>(smem + S::OFF_DKEY);
  void** dpay                 = reinterpret_cast<void**>(smem + S::OFF_DPAY);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < nbp - 1) ssplit[tid] = split[tid];
  if (tid < nbp) {
    goff[tid] = tile_off[(size_t)blockIdx.x * nbp + tid];
    dkey[tid] = dst.keys[tid];
    dpay[tid] = dst.pay[tid];
  }
  for (int i = tid; i < PART_WARPS * MAX_BUCKETS; i += PART_THREADS) wcnt[i] = 0;
  __syncthreads();

  const long long base = (long long)blockIdx.x * PART_TILE;
  const int valid      = (int)min((long long)PART_TILE, n - base);
  // a warp owns PART_ITEMS * 32 consecutive elements; element i of lane l sits at 32 * i + l of them
  const int stripe0 = warp * (PART_ITEMS * 32) + lane;
  Raw key[PART_ITEMS];
  unsigned int br[PART_ITEMS];  // bucket (bits 24..31) and rank among the warp's elements of that bucket
  unsigned int* my_cnt  = wcnt + warp * MAX_BUCKETS;
  const unsigned int lt = lanemask_lt();
  // all loads of the thread are issued before the first use, so that their latencies overlap
#pragma unroll
  for (int i = 0; i < PART_ITEMS; ++i) {
    const int e = stripe0 + 32 * i;
    if (e < valid) key[i] = keys[base + e];
  }
#pragma unroll
  for (int i = 0; i < PART_ITEMS; ++i) {
    const int e    = stripe0 + 32 * i;
    unsigned int b = NO_BUCKET;
    if (e < valid) b = classify(ssplit, nbp - 1, DKey<KB>::okey(key[i], xf), base + e);
    const unsigned int peers = __match_any_sync(0xFFFFFFFFu, b);
    unsigned int old         = 0;
    if (b != NO_BUCKET) old = my_cnt[b];
    __syncwarp();
    if (b != NO_BUCKET) my_cnt[b] = old + __popc(peers);  // the same value from every lane of the group
    __syncwarp();
    br[i] = (b << 24) | (old + __popc(peers & lt));
  }
  __syncthreads();
  // per bucket: exclusive prefix over the warps, then over the buckets (one warp)
  if (tid < 32) {
    unsigned int run = 0;
    if (tid < nbp) {
      for (int w = 0; w < PART_WARPS; ++w) {
        const unsigned int t        = wcnt[w * MAX_BUCKETS + tid];
        wcnt[w * MAX_BUCKETS + tid] = run;
        run += t;
      }
    }
    unsigned int incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    bstart[tid] = incl - run;
    if (tid == 31) bstart[32] = incl;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < PART_ITEMS; ++i) {
    const unsigned int b = br[i] >> 24;
    if (b != NO_BUCKET) {
      const unsigned int p = bstart[b] + my_cnt[b] + (br[i] & 0xFFFFFFu);
      skeys[p]             = key[i];
      const long long g    = global_offset + base + stripe0 + 32 * i;
      if (PAYB == 4) reinterpret_cast<uint32_t*>(spay)[p] = (uint32_t)(g - pay_base);
      if (PAYB == 8) reinterpret_cast<int64_t*>(spay)[p] = (int64_t)g;
    }
  }
  __syncthreads();
  // copy-out: staged position p belongs to the bucket whose range [bstart[b], bstart[b+1]) holds it
  for (int p = tid; p < valid; p += PART_THREADS) {
    int lo = 0, hi = nbp - 1;  // largest b with bstart[b] <= p
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (bstart[mid] <= (unsigned int)p) lo = mid; else hi = mid - 1;
    }
    const unsigned long long at = goff[lo] + (unsigned int)(p - bstart[lo]);
    static_cast<Raw*>(dkey[lo])[at] = skeys[p];
    if (PAYB == 4) static_cast<uint32_t*>(dpay[lo])[at] = reinterpret_cast<const uint32_t*>(spay)[p];
    if (PAYB == 8) static_cast<int64_t*>(dpay[lo])[at] = reinterpret_cast<const int64_t*>(spay)[p];
  }
}

// result[i] = payload[position[i]] (+ base for 32-bit payloads): turns an argsort of the receive
// buffer into global indices when the radix passes could not carry the payload themselves.
template <typename P>
__global__ void gather_payload_kernel(const int64_t* __restrict__ position, const P* __restrict__ payload, long long n,
                                      long long base, int64_t* __restrict__ result)
{
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    result[i] = (int64_t)payload[position[i]] + base;
}

template <typename F>
static cudaError_t by_width(int kb, F&& f)
{
  switch (kb) {
    case 1: return f(std::integral_constant<int, 1>{});
    case 2: return f(std::integral_constant<int, 2>{});
    case 4: return f(std::integral_constant<int, 4>{});
    default: return f(std::integral_constant<int, 8>{});
  }
}
template <typename F>
static cudaError_t by_width16(int kb, F&& f)
{
  if (kb == 16) return f(std::integral_constant<int, 16>{});
  return by_width(kb, f);
}

// Memory from the caller's allocator that goes back to it when the call ends, unless disowned.
struct Scratch {
  b2s_alloc_fn alloc;
  b2s_free_fn release;
  void* ctx;
  std::vector<void*> owned;
  void* get(size_t bytes)
  {
    void* p = alloc(ctx, bytes ? bytes : 256);
    if (p) owned.push_back(p);
    return p;
  }
  void drop(void* p)
  {
    for (auto& q : owned)
      if (q == p) { q = nullptr; }
    if (p && release) release(ctx, p);
  }
  // keep `p` alive past the call (ownership passes to the caller)
  void disown(void* p)
  {
    for (auto& q : owned)
      if (q == p) q = nullptr;
  }
  ~Scratch()
  {
    for (void* q : owned)
      if (q && release) release(ctx, q);
  }
};

// Launches the partition and merge kernels for `runs` (total elements) into `out`.
// probes per search step (minus one) in the two partition launches: the coarse one has few,
// long searches and is pure latency; the fine one has many short ones
#ifndef B2S_PART_ARY_COARSE
#define B2S_PART_ARY_COARSE 8
#endif
#ifndef B2S_PART_ARY_FINE
#define B2S_PART_ARY_FINE 2
#endif

static int merge_runs(int kb, int xf, const MergeRuns& runs, long long total, bool args, void* out,
                      long long* d_tcuts, cudaStream_t stream)
{
  const long long ntiles = (total + MERGE_TILE - 1) / MERGE_TILE;
  cudaError_t e = by_width(kb, [&](auto w) {
    constexpr int KB = decltype(w)::value;
    {
      prof::Scope ps(prof::K_DIST, stream);
      const long long ncoarse = (ntiles + MERGE_COARSE_STRIDE - 1) / MERGE_COARSE_STRIDE + 1;
      int gw = 1;
      while (gw < runs.nruns) gw <<= 1;
      const long long per_cta = 8 * (32 / gw);  // boundaries per CTA of 8 warps
      merge_partition_kernel<KB, B2S_PART_ARY_COARSE><<<(unsigned int)((ncoarse + per_cta - 1) / per_cta), 256, 0, stream>>>(
        runs, total, ntiles, xf, d_tcuts, MERGE_COARSE_STRIDE, 0);
    }
    {
      prof::Scope ps(prof::K_DIST, stream);
      const long long warps = ntiles + 1;
      int gw = 1;
      while (gw < runs.nruns) gw <<= 1;
      const long long per_cta = 8 * (32 / gw);
      merge_partition_kernel<KB, B2S_PART_ARY_FINE><<<(unsigned int)((warps + per_cta - 1) / per_cta), 256, 0, stream>>>(
        runs, total, ntiles, xf, d_tcuts, MERGE_COARSE_STRIDE, 1);
    }
    prof::Scope ps(prof::K_MERGE, stream);
    auto launch = [&](auto kern, size_t bytes) {
      cudaError_t ee = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
      if (ee != cudaSuccess) return ee;
      kern<<<(unsigned int)ntiles, MERGE_THREADS, bytes, stream>>>(runs, total, xf, d_tcuts, out);
      return cudaSuccess;
    };
    const bool flt = xf == XF_FLOAT || xf == XF_CFLOAT;  // ordered image cannot be mapped back
    cudaError_t ee;
    if (args && flt) ee = launch(merge_tiles_kernel<KB, true, true>, MergeSmem<KB, true, true>::BYTES);
    else if (args) ee = launch(merge_tiles_kernel<KB, true, false>, MergeSmem<KB, true, false>::BYTES);
    else if (flt) ee = launch(merge_tiles_kernel<KB, false, true>, MergeSmem<KB, false, true>::BYTES);
    else ee = launch(merge_tiles_kernel<KB, false, false>, MergeSmem<KB, false, false>::BYTES);
    if (ee != cudaSuccess) return ee;
    return cudaGetLastError();
  });
  return e == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
}

// Host-side phase trace of the distributed sort (B2S_DIST_TRACE=1, rank 0 prints; "a": all ranks).
struct PhaseTrace {
  bool on;
  int rk;
  std::chrono::steady_clock::time_point t0;
  char line[512] = {0};
  int used = 0;
  explicit PhaseTrace(int rank)
    : on(std::getenv("B2S_DIST_TRACE") != nullptr && (rank == 0 || std::getenv("B2S_DIST_TRACE")[0] == 'a')), rk(rank),
      t0(std::chrono::steady_clock::now()) {}
  // "s" as the second character of the value waits for the stream first, so that the figures are
  // device times per phase instead of enqueue times
  void mark(const char* what, cudaStream_t stream = nullptr)
  {
    if (!on) return;
    const char* e = std::getenv("B2S_DIST_TRACE");
    if (e != nullptr && e[0] != 0 && e[1] == 's') cudaStreamSynchronize(stream);
    const auto t1 = std::chrono::steady_clock::now();
    if (used < (int)sizeof(line) - 1) {
      const int w = std::snprintf(line + used, sizeof(line) - used, " %s=%.2f", what,
                                  std::chrono::duration<double, std::milli>(t1 - t0).count());
      if (w > 0) used = used + w < (int)sizeof(line) ? used + w : (int)sizeof(line) - 1;
    }
    t0 = t1;
  }
  ~PhaseTrace() { if (on) std::fprintf(stderr, "[b2s dist ms r%d]%s\n", rk, line); }
};

// One CUDA event that is destroyed on every way out of the function that owns it.
struct Event {
  cudaEvent_t ev = nullptr;
  Event() { if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) ev = nullptr; }
  ~Event() { if (ev) cudaEventDestroy(ev); }
};

// For rare failures inside the distributed calls: a local CUDA error is recorded and the rank
// keeps taking part in every collective, so that no other rank is left waiting for it.
struct Status {
  int code = B2S_OK;
  void cuda(cudaError_t e) { if (e != cudaSuccess && code == B2S_OK) code = B2S_ERR_CUDA; }
  void set(int rc) { if (rc != B2S_OK && code == B2S_OK) code = rc; }
  bool ok() const { return code == B2S_OK; }
};

// Used by the collectives of a rank whose control allocation failed: it has no memory of its own
// to take part with, and taking part is what keeps the others from waiting for ever.  The contents
// are never looked at (the rank's status says it failed).
constexpr size_t EMERGENCY_BYTES = sizeof(BlockA) * (MAX_BUCKETS + 1);
static __device__ __align__(256) unsigned char g_emergency[EMERGENCY_BYTES];

static unsigned char* emergency_area()
{
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_emergency) != cudaSuccess) return nullptr;
  return static_cast<unsigned char*>(p);
}

static size_t single_limit()
{
  // the same rule as the local sort's (a testing aid lowers it)
  const char* e = std::getenv("B2S_MAX_1D_LOG2");
  if (e != nullptr) {
    const int v = std::atoi(e);
    if (v >= 10 && v <= 30) return (size_t)1 << v;
  }
  return (size_t)1 << 30;
}

}  // namespace b2s

using namespace b2s;

extern "C" {

// ---- host-side pieces, exported so that they can be exercised without a GPU -----------------
void b2s_host_sort_samples(void* samples, size_t count)
{
  Sample* s = static_cast<Sample*>(samples);
  std::stable_sort(s, s + count, [](const Sample& a, const Sample& b) { return sample_less(a, b); });
}

int b2s_host_select_splitters(void* samples, size_t count, int nbuckets, void* splitters_out)
{
  if (samples == nullptr || splitters_out == nullptr || nbuckets < 1 || nbuckets > MAX_BUCKETS) return B2S_ERR_INVALID_ARG;
  Sample* s   = static_cast<Sample*>(samples);
  Sample* out = static_cast<Sample*>(splitters_out);
  b2s_host_sort_samples(s, count);
  long long total = 0;
  for (size_t t = 0; t < count; ++t) total += s[t].weight;
  for (int k = 1; k < nbuckets; ++k) {
    Sample sp{};
    sp.okey = OKey{~0ull, ~0ull};
    if (total > 0) {
      const long long target = splitter_target(k, total, nbuckets);
      long long run = 0;
      for (size_t t = 0; t < count; ++t) {
        run += s[t].weight;
        if (run >= target) {
          sp = s[t];
          break;
        }
      }
    }
    out[k - 1] = sp;
  }
  return B2S_OK;
}

long long b2s_host_sample_position(long long j, long long s, long long n) { return sample_position(j, s, n); }
long long b2s_host_sample_weight(long long j, long long s, long long n) { return sample_weight(j, s, n); }

int b2s_host_bucket_of(const void* splitters, int nsplit, int my_rank, unsigned long long okey_hi, unsigned long long okey_lo,
                       long long pos)
{
  if (nsplit < 0 || nsplit >= MAX_BUCKETS || (nsplit > 0 && splitters == nullptr)) return -1;
  LocalSplitter local[MAX_BUCKETS];
  const Sample* sp = static_cast<const Sample*>(splitters);
  for (int k = 0; k < nsplit; ++k) local[k] = localise(sp[k], my_rank);
  return bucket_of(local, nsplit, OKey{okey_hi, okey_lo}, pos);
}

int b2s_samples_per_rank(void) { return SAMPLES_PER_RANK; }

// ---- k-way merge ---------------------------------------------------------------------------
int b2s_kway_merge_workspace_bytes(size_t total, int nruns, size_t* bytes)
{
  if (bytes == nullptr || nruns < 1 || nruns > MERGE_MAX_RUNS) return B2S_ERR_INVALID_ARG;
  const size_t ntiles = (total + MERGE_TILE - 1) / MERGE_TILE;
  *bytes              = align_up(sizeof(long long) * (ntiles + 1) * nruns, 256);
  return B2S_OK;
}

int b2s_kway_merge(int dtype, int nruns, const void* const* run_keys, const int64_t* const* run_idx,
                   const size_t* run_len, void* out, void* ws, size_t ws_bytes, void* cuda_stream)
{
  int xf       = 0;
  const int kb = kb_of(dtype, &xf);
  if (kb == 0 || kb == 16) return B2S_ERR_UNSUPPORTED;
  if (nruns < 1 || nruns > MERGE_MAX_RUNS || run_keys == nullptr || run_len == nullptr) return B2S_ERR_INVALID_ARG;
  MergeRuns runs{};
  runs.nruns      = nruns;
  long long total = 0;
  for (int i = 0; i < nruns; ++i) {
    runs.keys[i] = run_keys[i];
    runs.idx[i]       = run_idx ? run_idx[i] : nullptr;
    runs.idx_bytes[i] = 8;
    runs.idx_base[i]  = 0;
    runs.len[i]  = (long long)run_len[i];
    if (run_len[i] > 0 && (run_keys[i] == nullptr || (run_idx && run_idx[i] == nullptr))) return B2S_ERR_INVALID_ARG;
    total += runs.len[i];
  }
  if (total == 0) return B2S_OK;
  size_t need = 0;
  b2s_kway_merge_workspace_bytes((size_t)total, nruns, &need);
  if (out == nullptr) return B2S_ERR_INVALID_ARG;
  if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 7u)) return B2S_ERR_WORKSPACE;
  return merge_runs(kb, xf, runs, total, run_idx != nullptr, out, static_cast<long long*>(ws),
                    static_cast<cudaStream_t>(cuda_stream));
}

// ---- NCCL communicator plumbing --------------------------------------------------------------
int b2s_nccl_unique_id(void* out128)
{
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  if (out128 == nullptr) return B2S_ERR_INVALID_ARG;
  return ncclGetUniqueId(static_cast<ncclUniqueId*>(out128)) == ncclSuccess ? B2S_OK : B2S_ERR_NCCL;
}

int b2s_nccl_comm_create(void** comm, int nranks, const void* id128, int rank)
{
  if (comm == nullptr || id128 == nullptr) return B2S_ERR_INVALID_ARG;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t c;
  if (ncclCommInitRank(&c, nranks, id, rank) != ncclSuccess) return B2S_ERR_NCCL;
  *comm = c;
  return B2S_OK;
}

int b2s_nccl_comm_destroy(void* comm)
{
  if (comm == nullptr) return B2S_OK;
  return ncclCommDestroy(static_cast<ncclComm_t>(comm)) == ncclSuccess ? B2S_OK : B2S_ERR_NCCL;
}

// ---- rebalance -----------------------------------------------------------------------------
int b2s_dist_rebalance_1d_ops(size_t elem_bytes, const void* part, size_t part_len, int64_t part_global_start,
                              void* out, size_t out_len, int64_t out_global_start, const b2s_comm_ops* ops, int rank,
                              int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                              b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream)
{
  if (elem_bytes == 0 || nranks < 1 || nranks > MAX_BUCKETS || rank < 0 || rank >= nranks || alloc == nullptr)
    return B2S_ERR_INVALID_ARG;
  if ((part_len > 0 && part == nullptr) || (out_len > 0 && out == nullptr)) return B2S_ERR_INVALID_ARG;
  if (nranks > 1 && ops == nullptr) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  Scratch mem{alloc, release, alloc_ctx, {}};
  Status st;
  // every rank learns where every rank's sorted part and output extent lie in the global order,
  // and whether it got this far in one piece
  long long mine[8] = {(long long)part_global_start, (long long)part_len, (long long)out_global_start, (long long)out_len, 0, 0, 0, 0};
  std::vector<long long> all((size_t)8 * nranks);
  if (nranks == 1) {
    std::copy(mine, mine + 8, all.begin());
  } else {
    long long* d_all = static_cast<long long*>(mem.get(sizeof(long long) * 8 * (nranks + 1)));
    if (d_all == nullptr) {
      st.set(B2S_ERR_WORKSPACE);
      d_all = reinterpret_cast<long long*>(emergency_area());
      if (d_all == nullptr) return B2S_ERR_CUDA;  // no device memory at all to take part with
    }
    mine[4] = st.code;
    st.cuda(cudaMemcpyAsync(d_all + 8 * nranks, mine, sizeof(mine), cudaMemcpyHostToDevice, stream));
    if (barrier) barrier(barrier_ctx);
    st.set(ops->all_gather(ops->ctx, d_all + 8 * nranks, d_all, sizeof(mine), stream));
    if (barrier) barrier(barrier_ctx);
    st.cuda(cudaMemcpyAsync(all.data(), d_all, sizeof(long long) * 8 * nranks, cudaMemcpyDeviceToHost, stream));
    st.cuda(cudaStreamSynchronize(stream));
    if (!st.ok()) return st.code;  // nothing the others sent can be trusted either
  }
  long long parts_total = 0, outs_total = 0;
  int worst = B2S_OK;
  for (int p = 0; p < nranks; ++p) {
    parts_total += all[8 * p + 1];
    outs_total += all[8 * p + 3];
    if (all[8 * p + 4] != B2S_OK) worst = (int)all[8 * p + 4];
  }
  if (worst != B2S_OK) return worst;                            // every rank sees the same flags
  if (parts_total != outs_total) return B2S_ERR_INVALID_ARG;    // extents must tile what was sorted
  const unsigned char* src = static_cast<const unsigned char*>(part);
  unsigned char* dst       = static_cast<unsigned char*>(out);
  auto overlap = [](long long a0, long long a1, long long b0, long long b1, long long* lo, long long* hi) {
    *lo = a0 > b0 ? a0 : b0;
    *hi = a1 < b1 ? a1 : b1;
    return *hi > *lo;
  };
  const long long ps = mine[0], pe = mine[0] + mine[1], os = mine[2], oe = mine[2] + mine[3];
  if (nranks > 1) {
    std::vector<const void*> sp(nranks, nullptr);
    std::vector<void*> rp(nranks, nullptr);
    std::vector<size_t> sb(nranks, 0), rb(nranks, 0);
    for (int p = 0; p < nranks; ++p) {
      if (p == rank) continue;
      long long lo, hi;
      if (overlap(ps, pe, all[8 * p + 2], all[8 * p + 2] + all[8 * p + 3], &lo, &hi)) {
        sp[p] = src + (size_t)(lo - ps) * elem_bytes;
        sb[p] = (size_t)(hi - lo) * elem_bytes;
      }
      if (overlap(all[8 * p], all[8 * p] + all[8 * p + 1], os, oe, &lo, &hi)) {
        rp[p] = dst + (size_t)(lo - os) * elem_bytes;
        rb[p] = (size_t)(hi - lo) * elem_bytes;
      }
    }
    if (barrier) barrier(barrier_ctx);
    st.set(ops->exchange(ops->ctx, sp.data(), sb.data(), rp.data(), rb.data(), stream));
    if (barrier) barrier(barrier_ctx);
  }
  long long lo, hi;
  if (overlap(ps, pe, os, oe, &lo, &hi))
    st.cuda(cudaMemcpyAsync(dst + (size_t)(lo - os) * elem_bytes, src + (size_t)(lo - ps) * elem_bytes,
                            (size_t)(hi - lo) * elem_bytes, cudaMemcpyDeviceToDevice, stream));
  st.cuda(cudaStreamSynchronize(stream));
  return st.code;
}

// ---- the distributed sort ---------------------------------------------------------------------
int b2s_dist_sort_1d_ops(int dtype, const void* keys_in, size_t n_local, int64_t global_offset, int argsort,
                         const b2s_comm_ops* ops, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                         void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void** out_ptr,
                         size_t* out_len, int64_t* out_global_offset, void* cuda_stream)
{
  int xf       = 0;
  const int kb = kb_of(dtype, &xf);
  if (kb == 0) return B2S_ERR_UNSUPPORTED;
  if (alloc == nullptr || out_ptr == nullptr || out_len == nullptr || nranks < 1 || rank < 0 || rank >= nranks)
    return B2S_ERR_INVALID_ARG;
  if (nranks > MAX_BUCKETS) return B2S_ERR_UNSUPPORTED;
  if (nranks > 1 && (ops == nullptr || ops->all_gather == nullptr || ops->barrier == nullptr || ops->exchange == nullptr))
    return B2S_ERR_INVALID_ARG;
  if (n_local > 0 && keys_in == nullptr) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  Scratch mem{alloc, release, alloc_ctx, {}};
  const long long n = (long long)n_local;
  const size_t out_elem = argsort ? 8 : (size_t)kb;
  PhaseTrace trace(rank);

  // ---- one rank: the local sort, result in allocator memory ----
  if (nranks == 1) {
    void* result = mem.get(n_local * out_elem);
    if (result == nullptr) return B2S_ERR_WORKSPACE;
    if (n > 0) {
      size_t ws_bytes = 0;
      int rc = b2s_workspace_bytes(dtype, n_local, n_local, argsort, &ws_bytes);
      if (rc != B2S_OK) return rc;
      void* ws = mem.get(ws_bytes);
      if (ws == nullptr) return B2S_ERR_WORKSPACE;
      rc = b2s_local_sort(dtype, keys_in, argsort ? nullptr : result, argsort ? static_cast<int64_t*>(result) : nullptr, n_local,
                          n_local, global_offset, 1, 1, ws, ws_bytes, stream);
      if (rc != B2S_OK) return rc;
      rc = dtype == B2S_COMPLEX128 ? (cudaStreamSynchronize(stream) == cudaSuccess ? B2S_OK : B2S_ERR_CUDA)
                                   : b2s_check_status(ws, stream);
      if (rc != B2S_OK) return rc;
    }
    mem.disown(result);
    *out_ptr = result;
    *out_len = n_local;
    if (out_global_offset) *out_global_offset = 0;
    return B2S_OK;
  }

  // From here on every rank goes through every collective, whatever happens to it locally: its
  // status travels with the gathered blocks and all ranks return a failure together.
  Status st;
  const int nb  = nranks;
  // up to 8 destinations and keys of at most 8 bytes: the register-counting partition kernels
  const bool fast = nb <= FP_NB && kb <= 8;
  // With the register-counting kernels the counting pass can also count, per destination, the digits
  // of the keys it will send there; every destination gets the tables of what it receives and its
  // local sort starts without reading its keys for a histogram.  Only with B2S_DIST_SENDER_HIST=1:
  // measured on 8 GPUs (2^28 keys each) the counting pass grows by more than the histogram pass it
  // saves (float32: 1.62 vs 0.59 + 0.49 ms, int64: 2.27 vs 0.66 + 0.87 ms), and counting inside the
  // partition kernel instead was worse still (its tables cut the CTAs per SM and with them the
  // stores in flight towards NVLink).
  const char* sh_env    = std::getenv("B2S_DIST_SENDER_HIST");
  const bool count_hist = fast && nranks > 1 && sh_env != nullptr && sh_env[0] == '1';
  int nbp         = 1;
  while (nbp < nb) nbp <<= 1;                       // padded bucket count
  if (fast) nbp = FP_NB;
  const int S_all            = nranks * SAMPLES_PER_RANK;
  const long long ntiles     = (n + PART_TILE - 1) / PART_TILE;
  const long long capacity   = n + n / 8 + 65536;  // elements my receive buffers hold
  const size_t pay_cap_bytes = argsort ? 8 : 0;     // per element, enough for either payload width

  // ---- control block: one allocation ----
  size_t off = 0;
  auto take  = [&](size_t bytes) { const size_t at = off; off += align_up(bytes, 256); return at; };
  const size_t o_mineA = take(sizeof(BlockA)), o_allA = take(sizeof(BlockA) * nranks);
  const size_t o_samples = take(sizeof(Sample) * S_all), o_khi = take(8 * (size_t)S_all), o_klo = take(8 * (size_t)S_all);
  const size_t o_tmp = take(8 * (size_t)S_all), o_ord1 = take(8 * (size_t)S_all), o_ord2 = take(8 * (size_t)S_all);
  const size_t o_cum = take(8 * (size_t)S_all), o_split = take(sizeof(Sample) * MAX_BUCKETS);
  const size_t o_local = take(sizeof(LocalSplitter) * MAX_BUCKETS);
  const size_t o_counts = take(4 * (size_t)(ntiles > 0 ? ntiles : 1) * nbp), o_toff = take(8 * (size_t)(ntiles > 0 ? ntiles : 1) * nbp);
  const size_t o_totals = take(8 * MAX_BUCKETS), o_mineB = take(sizeof(BlockB)), o_allB = take(sizeof(BlockB) * nranks);
  const long long nchunks = (ntiles + FP_CHUNK_TILES - 1) / FP_CHUNK_TILES;
  // zeroed together: the partition kernels' status word and the per-chunk sums of the tile counts
  constexpr size_t SENT_BYTES = (size_t)FP_NB * 8 * RADIX * 4;
  const size_t zero_bytes = 256 + SENT_BYTES + 8 * (size_t)FP_NB * (size_t)(nchunks > 0 ? nchunks : 1);
  const size_t o_zero     = take(zero_bytes);
  size_t sample_ws_bytes = 0;
  b2s_workspace_bytes(B2S_UINT64, (size_t)S_all, (size_t)S_all, 1, &sample_ws_bytes);
  const size_t o_sws = take(sample_ws_bytes);
  unsigned char* ctl = static_cast<unsigned char*>(mem.get(off));
  bool have_ctl      = ctl != nullptr;
  if (!have_ctl) {
    st.set(B2S_ERR_WORKSPACE);
    ctl = emergency_area();
    if (ctl == nullptr) return B2S_ERR_CUDA;  // not even the library's own device memory answers
  }
  // receive buffers the other ranks write into; in front of the keys a landing area for the digit
  // histograms of what every rank sends here (one [8][256] table of counts per source rank)
  constexpr size_t LANDING_BYTES = (size_t)MAX_BUCKETS * 8 * RADIX * 4;
  unsigned char* recv_block = have_ctl ? static_cast<unsigned char*>(mem.get(LANDING_BYTES + (size_t)capacity * kb + 256)) : nullptr;
  void* recv_keys = recv_block ? recv_block + LANDING_BYTES : nullptr;
  void* recv_pay  = (have_ctl && argsort) ? mem.get((size_t)capacity * pay_cap_bytes + 256) : nullptr;
  if (have_ctl && (recv_keys == nullptr || (argsort && recv_pay == nullptr))) st.set(B2S_ERR_WORKSPACE);

  BlockA* d_mineA = reinterpret_cast<BlockA*>(ctl + (have_ctl ? o_mineA : 0));
  BlockA* d_allA  = reinterpret_cast<BlockA*>(ctl + (have_ctl ? o_allA : sizeof(BlockA)));
  BlockA h_mineA{};
  h_mineA.n_local       = n;
  h_mineA.global_offset = global_offset;
  h_mineA.capacity      = capacity;
  {
    void* bufs[PEER_BUFFERS] = {recv_block, recv_pay};
    export_buffers(bufs, argsort ? 2 : 1, &h_mineA.rec);
    if (!st.ok()) h_mineA.rec.ok = 0;
  }
  h_mineA.status = st.code;
  // header first, then the samples straight into the block on the device
  st.cuda(cudaMemcpyAsync(d_mineA, &h_mineA, offsetof(BlockA, okey), cudaMemcpyHostToDevice, stream));
  if (st.ok()) {
    prof::Scope ps(prof::K_DIST, stream);
    by_width16(kb, [&](auto w) {
      constexpr int KB = decltype(w)::value;
      sample_kernel<KB><<<(SAMPLES_PER_RANK + 255) / 256, 256, 0, stream>>>(
        static_cast<const typename DKey<KB>::Raw*>(keys_in), n, xf, d_mineA->okey);
      return cudaSuccess;
    });
    st.cuda(cudaGetLastError());
  }
  if (barrier) barrier(barrier_ctx);
  st.set(ops->all_gather(ops->ctx, d_mineA, d_allA, sizeof(BlockA), stream));
  if (barrier) barrier(barrier_ctx);
  // the headers come to the host while the device goes on with the splitters
  std::vector<BlockA> h_allA_hdr(nranks);
  std::vector<unsigned char> h_hdr((size_t)nranks * offsetof(BlockA, okey));
  st.cuda(cudaMemcpy2DAsync(h_hdr.data(), offsetof(BlockA, okey), d_allA, sizeof(BlockA), offsetof(BlockA, okey), nranks,
                            cudaMemcpyDeviceToHost, stream));
  Event ev_hdr;
  if (ev_hdr.ev == nullptr) st.set(B2S_ERR_CUDA); else st.cuda(cudaEventRecord(ev_hdr.ev, stream));
  trace.mark("samples", stream);

  // ---- splitters on the device: order the samples by (key, rank, position), weigh, pick ----
  Sample* d_samples     = reinterpret_cast<Sample*>(ctl + o_samples);
  LocalSplitter* d_local = reinterpret_cast<LocalSplitter*>(ctl + o_local);
  unsigned int* d_counts = reinterpret_cast<unsigned int*>(ctl + o_counts);
  unsigned long long* d_toff = reinterpret_cast<unsigned long long*>(ctl + o_toff);
  long long* d_totals    = reinterpret_cast<long long*>(ctl + o_totals);
  unsigned int* d_status = reinterpret_cast<unsigned int*>(ctl + (have_ctl ? o_zero : 0));
  unsigned long long* d_chunks = reinterpret_cast<unsigned long long*>(ctl + o_zero + 256 + SENT_BYTES);
  unsigned int* d_sent         = reinterpret_cast<unsigned int*>(ctl + o_zero + 256);  // [FP_NB][kb][256] digit counts per destination
  if (have_ctl) st.cuda(cudaMemsetAsync(ctl + o_zero, 0, zero_bytes, stream));
  if (have_ctl && st.ok()) {
    unsigned long long* khi = reinterpret_cast<unsigned long long*>(ctl + o_khi);
    unsigned long long* klo = reinterpret_cast<unsigned long long*>(ctl + o_klo);
    unsigned long long* tmp = reinterpret_cast<unsigned long long*>(ctl + o_tmp);
    int64_t* ord1 = reinterpret_cast<int64_t*>(ctl + o_ord1);
    int64_t* ord2 = reinterpret_cast<int64_t*>(ctl + o_ord2);
    int64_t* order = ord1;
    prof::Account sample_sort_is_bookkeeping(prof::K_DIST);
    {
      prof::Scope ps(prof::K_DIST, stream);
      build_samples_kernel<<<(S_all + 255) / 256, 256, 0, stream>>>(d_allA, nranks, d_samples, khi, klo);
    }
    if (kb == 16) {
      // two-word keys: stable order by the minor word, then by the major one
      st.set(b2s_local_sort(B2S_UINT64, klo, nullptr, ord1, (size_t)S_all, (size_t)S_all, 0, 1, 1, ctl + o_sws, sample_ws_bytes, stream));
      {
        prof::Scope ps(prof::K_DIST, stream);
        gather_u64_kernel<<<(S_all + 255) / 256, 256, 0, stream>>>(khi, ord1, S_all, tmp);
      }
      st.set(b2s_local_sort(B2S_UINT64, tmp, nullptr, ord2, (size_t)S_all, (size_t)S_all, 0, 1, 1, ctl + o_sws, sample_ws_bytes, stream));
      {
        prof::Scope ps(prof::K_DIST, stream);
        compose_kernel<<<(S_all + 255) / 256, 256, 0, stream>>>(ord1, ord2, S_all, reinterpret_cast<int64_t*>(tmp));
      }
      order = reinterpret_cast<int64_t*>(tmp);
    } else {
      st.set(b2s_local_sort(B2S_UINT64, khi, nullptr, ord1, (size_t)S_all, (size_t)S_all, 0, 1, 1, ctl + o_sws, sample_ws_bytes, stream));
    }
    {
      prof::Scope ps(prof::K_DIST, stream);
      select_splitters_kernel<<<1, SELECT_THREADS, 0, stream>>>(d_samples, order, S_all, nb, rank,
                                                                reinterpret_cast<long long*>(ctl + o_cum),
                                                                reinterpret_cast<Sample*>(ctl + o_split), d_local, nbp - 1 > 0 ? nbp - 1 : 1);
    }
    // ---- count my elements per destination ----
    if (n > 0) {
      {
        prof::Scope ps(prof::K_DIST, stream);
        if (fast && count_hist) {
          by_width(kb, [&](auto w) {
            constexpr int KB     = decltype(w)::value;
            constexpr size_t TAB = (size_t)FP_NB * KB * RADIX * 4;
            auto kern            = part_count_hist_kernel<KB>;
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TAB);
            if (e != cudaSuccess) return e;
            int dev = 0, sms = 148, per_sm = 1;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, FP_THREADS, TAB);
            const long long grid = std::min<long long>(ntiles, (long long)sms * (per_sm < 1 ? 1 : per_sm));
            kern<<<(unsigned int)grid, FP_THREADS, TAB, stream>>>(static_cast<const typename FpKey<KB>::Raw*>(keys_in), n, ntiles, xf,
                                                                    d_local, d_counts, d_chunks, d_sent);
            return cudaGetLastError();
          });
        } else if (fast) {
          by_width(kb, [&](auto w) {
            constexpr int KB = decltype(w)::value;
            part_count_fast_kernel<KB><<<(unsigned int)ntiles, FP_THREADS, 0, stream>>>(
              static_cast<const typename FpKey<KB>::Raw*>(keys_in), n, xf, d_local, d_counts, d_chunks);
            return cudaSuccess;
          });
        } else {
          by_width16(kb, [&](auto w) {
            constexpr int KB = decltype(w)::value;
            part_count_kernel<KB><<<(unsigned int)ntiles, PART_THREADS, 0, stream>>>(
              static_cast<const typename DKey<KB>::Raw*>(keys_in), n, xf, d_local, nbp, d_counts);
            return cudaSuccess;
          });
        }
      }
      {
        prof::Scope ps(prof::K_DIST, stream);
        if (fast)
          tile_scan_fast_kernel<<<(unsigned int)nchunks, FP_NB * 32, 0, stream>>>(d_counts, ntiles, d_chunks, d_toff, d_totals);
        else
          tile_scan_kernel<<<nbp, SCAN_THREADS, 0, stream>>>(d_counts, ntiles, nbp, d_toff, d_totals);
      }
    } else {
      st.cuda(cudaMemsetAsync(d_totals, 0, 8 * MAX_BUCKETS, stream));
    }
    st.cuda(cudaGetLastError());
  }

  // ---- meanwhile on the host: who can write where ----
  if (ev_hdr.ev != nullptr) st.cuda(cudaEventSynchronize(ev_hdr.ev)); else st.cuda(cudaStreamSynchronize(stream));
  for (int p = 0; p < nranks; ++p) std::memcpy(&h_allA_hdr[p], &h_hdr[(size_t)p * offsetof(BlockA, okey)], offsetof(BlockA, okey));
  PeerPins pins;  // declared after `mem`: the mappings are let go before the buffers
  std::vector<unsigned char*> peer_keys(nranks, nullptr), peer_pay(nranks, nullptr);
  long long mapped = st.ok() ? 1 : 0;
  const unsigned long long my_pid = h_mineA.rec.pid;
  for (int p = 0; p < nranks && mapped; ++p) {
    const PeerRecord& r = h_allA_hdr[p].rec;
    if (!r.ok || r.nbuf != (unsigned long long)(argsort ? 2 : 1)) { mapped = 0; break; }
    if (p == rank) {
      peer_keys[p] = recv_block;
      peer_pay[p]  = static_cast<unsigned char*>(recv_pay);
    } else if (r.pid == my_pid) {
      if (!same_process_reachable((int)r.device)) { mapped = 0; break; }
      peer_keys[p] = reinterpret_cast<unsigned char*>((uintptr_t)r.ptr[0]);
      peer_pay[p]  = argsort ? reinterpret_cast<unsigned char*>((uintptr_t)r.ptr[1]) : nullptr;
    } else {
      unsigned char* kbase = static_cast<unsigned char*>(pins.acquire(r.handle[0]));
      unsigned char* pbase = argsort ? static_cast<unsigned char*>(pins.acquire(r.handle[1])) : nullptr;
      if (kbase == nullptr || (argsort && pbase == nullptr)) { mapped = 0; break; }
      peer_keys[p] = kbase + r.off[0];
      peer_pay[p]  = argsort ? pbase + r.off[1] : nullptr;
    }
  }
  // peer_keys[p] is rank p's receive block: landing area first, keys behind it
  std::vector<unsigned char*> peer_landing = peer_keys;
  for (int p = 0; p < nranks; ++p)
    if (peer_keys[p] != nullptr) peer_keys[p] += LANDING_BYTES;
  trace.mark("map", stream);

  // ---- second all-gather: counts per destination, mapping flag, status ----
  BlockB* d_mineB = reinterpret_cast<BlockB*>(ctl + (have_ctl ? o_mineB : 0));
  BlockB* d_allB  = reinterpret_cast<BlockB*>(ctl + (have_ctl ? o_allB : sizeof(BlockB)));
  {
    BlockB hb{};
    hb.status = st.code;
    hb.mapped = mapped;
    // the totals go from the device array straight into the block
    st.cuda(cudaMemcpyAsync(d_mineB, &hb, offsetof(BlockB, total), cudaMemcpyHostToDevice, stream));
    if (have_ctl) st.cuda(cudaMemcpyAsync(d_mineB->total, d_totals, 8 * MAX_BUCKETS, cudaMemcpyDeviceToDevice, stream));
  }
  if (barrier) barrier(barrier_ctx);
  st.set(ops->all_gather(ops->ctx, d_mineB, d_allB, sizeof(BlockB), stream));
  if (barrier) barrier(barrier_ctx);
  std::vector<BlockB> h_allB(nranks);
  st.cuda(cudaMemcpyAsync(h_allB.data(), d_allB, sizeof(BlockB) * nranks, cudaMemcpyDeviceToHost, stream));
  st.cuda(cudaStreamSynchronize(stream));
  trace.mark("count(sync)");
  if (!st.ok()) return st.code;  // my own copy failed: what I hold of the others cannot be trusted
  // Every rank sees the same blocks from here on, so every decision below is the same everywhere.
  {
    int worst = B2S_OK;
    for (int p = 0; p < nranks; ++p) {
      if (h_allA_hdr[p].status != B2S_OK) worst = (int)h_allA_hdr[p].status;
      if (h_allB[p].status != B2S_OK) worst = (int)h_allB[p].status;
    }
    if (worst != B2S_OK) return worst;
    for (int p = 0; p < nranks; ++p) {
      long long sum = 0;
      for (int b = 0; b < nb; ++b) {
        if (h_allB[p].total[b] < 0) return B2S_ERR_INVALID_ARG;  // protocol mismatch
        sum += h_allB[p].total[b];
      }
      if (sum != h_allA_hdr[p].n_local) return B2S_ERR_INVALID_ARG;
    }
  }
  std::vector<long long> recv_total(nranks, 0);
  std::vector<std::vector<long long>> recv_off(nranks, std::vector<long long>(nranks, 0));  // [dst][src]
  long long gmin = 0, gmax = 0, total_all = 0;
  bool any = false, direct = true;
  for (int d = 0; d < nranks; ++d) {
    for (int s = 0; s < nranks; ++s) {
      recv_off[d][s] = recv_total[d];
      recv_total[d] += h_allB[s].total[d];
    }
    if (recv_total[d] > h_allA_hdr[d].capacity) direct = false;  // a receive buffer is too small for direct writes
    if (!h_allB[d].mapped) direct = false;
    if (h_allA_hdr[d].n_local > 0) {
      const long long lo = h_allA_hdr[d].global_offset, hi = lo + h_allA_hdr[d].n_local;
      gmin = any ? std::min(gmin, lo) : lo;
      gmax = any ? std::max(gmax, hi) : hi;
      any  = true;
    }
    total_all += h_allA_hdr[d].n_local;
  }
  const long long n_recv = recv_total[rank];
  // payload of an argsort: global position minus the smallest one as 32 bits when that fits
  const int payb = !argsort ? 0 : ((gmax - gmin) <= 0xFFFFFFFFll ? 4 : 8);
  if (out_global_offset) {
    long long before = 0;
    for (int d = 0; d < rank; ++d) before += recv_total[d];
    *out_global_offset = before;
  }
  if (total_all == 0) {
    void* result = mem.get(256);
    if (result == nullptr) return B2S_ERR_WORKSPACE;
    mem.disown(result);
    *out_ptr = result;
    *out_len = 0;
    return B2S_OK;
  }

  // ---- partition my tile into the destinations' receive buffers ----
  void* send_keys = nullptr;
  void* send_pay  = nullptr;
  PartDst dst{};
  if (direct) {
    for (int d = 0; d < nranks; ++d) {
      dst.keys[d] = peer_keys[d] + (size_t)recv_off[d][rank] * kb;
      dst.pay[d]  = payb ? peer_pay[d] + (size_t)recv_off[d][rank] * payb : nullptr;
    }
  } else {
    // the collective exchange: partition into a local buffer (bucket after bucket), send from it
    send_keys = mem.get((size_t)n * kb + 256);
    send_pay  = payb ? mem.get((size_t)n * payb + 256) : nullptr;
    if (n_recv > capacity) {
      recv_keys = mem.get((size_t)n_recv * kb + 256);
      recv_pay  = payb ? mem.get((size_t)n_recv * payb + 256) : nullptr;
    }
    if (send_keys == nullptr || (payb && send_pay == nullptr) || recv_keys == nullptr || (payb && recv_pay == nullptr))
      st.set(B2S_ERR_WORKSPACE);
    long long at = 0;
    for (int d = 0; d < nranks; ++d) {
      dst.keys[d] = static_cast<unsigned char*>(send_keys) + (size_t)at * kb;
      dst.pay[d]  = payb ? static_cast<unsigned char*>(send_pay) + (size_t)at * payb : nullptr;
      at += h_allB[rank].total[d];
    }
    // one more agreement: a rank that could not allocate must not leave the others in the exchange
    long long* d_flag = reinterpret_cast<long long*>(d_mineB);
    const long long flag = st.code;
    std::vector<long long> flags(nranks * (sizeof(BlockB) / 8));
    st.cuda(cudaMemcpyAsync(d_flag, &flag, 8, cudaMemcpyHostToDevice, stream));
    if (barrier) barrier(barrier_ctx);
    st.set(ops->all_gather(ops->ctx, d_mineB, d_allB, sizeof(BlockB), stream));
    if (barrier) barrier(barrier_ctx);
    st.cuda(cudaMemcpyAsync(flags.data(), d_allB, sizeof(BlockB) * nranks, cudaMemcpyDeviceToHost, stream));
    st.cuda(cudaStreamSynchronize(stream));
    if (!st.ok()) return st.code;
    for (int p = 0; p < nranks; ++p)
      if (flags[p * (sizeof(BlockB) / 8)] != B2S_OK) return (int)flags[p * (sizeof(BlockB) / 8)];
  }
  const bool sender_hist = direct && count_hist;  // the tables were counted by the counting pass
  if (n > 0 && fast) {
    prof::Scope ps(prof::K_XCHG, stream);
    FpDst fd{};
    for (int d = 0; d < nranks; ++d) {
      fd.keys[d] = dst.keys[d];
      fd.pay[d]  = dst.pay[d];
    }
    by_width(kb, [&](auto w) {
      constexpr int KB = decltype(w)::value;
      using Raw        = typename FpKey<KB>::Raw;
      auto launch = [&](auto kern, size_t bytes) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        kern<<<(unsigned int)ntiles, FP_THREADS, bytes, stream>>>(static_cast<const Raw*>(keys_in), n, xf, d_local, d_toff, fd,
                                                                    (long long)global_offset, gmin, d_status);
        return cudaGetLastError();
      };
      if (payb == 0) return launch(part_scatter_fast_kernel<KB, 0>, FpSmem<KB, 0>::BYTES);
      if (payb == 4) return launch(part_scatter_fast_kernel<KB, 4>, FpSmem<KB, 4>::BYTES);
      return launch(part_scatter_fast_kernel<KB, 8>, FpSmem<KB, 8>::BYTES);
    });
    st.cuda(cudaGetLastError());
  }
  if (sender_hist) {
    // also from a rank with an empty tile: its (all-zero) table is what the others expect
    prof::Scope ps(prof::K_DIST, stream);
    FpDst land{};
    for (int d = 0; d < nranks; ++d) land.keys[d] = peer_landing[d];
    hist_deliver_kernel<<<nranks, 256, 0, stream>>>(d_sent, land, kb, rank);
    st.cuda(cudaGetLastError());
  }
  if (n > 0 && fast) {
  } else if (n > 0) {
    prof::Scope ps(prof::K_XCHG, stream);
    by_width16(kb, [&](auto w) {
      constexpr int KB = decltype(w)::value;
      using Raw        = typename DKey<KB>::Raw;
      auto launch = [&](auto kern, size_t bytes) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) return e;
        kern<<<(unsigned int)ntiles, PART_THREADS, bytes, stream>>>(static_cast<const Raw*>(keys_in), n, xf, d_local, nbp, d_toff,
                                                                      dst, (long long)global_offset, gmin);
        return cudaGetLastError();
      };
      if (payb == 0) return launch(part_scatter_kernel<KB, 0>, PartSmem<KB, 0>::BYTES);
      if (payb == 4) return launch(part_scatter_kernel<KB, 4>, PartSmem<KB, 4>::BYTES);
      return launch(part_scatter_kernel<KB, 8>, PartSmem<KB, 8>::BYTES);
    });
    st.cuda(cudaGetLastError());
  }
  if (direct) {
    // nobody reads its receive buffer before everybody has finished writing into it, and nobody
    // lets go of it before then either
    if (barrier) barrier(barrier_ctx);
    st.set(ops->barrier(ops->ctx, stream));
    if (barrier) barrier(barrier_ctx);
  } else {
    std::vector<const void*> sp(nranks, nullptr);
    std::vector<void*> rp(nranks, nullptr);
    std::vector<size_t> sb(nranks, 0), rb(nranks, 0);
    for (int pass = 0; pass < (payb ? 2 : 1); ++pass) {
      const size_t eb = pass == 0 ? (size_t)kb : (size_t)payb;
      unsigned char* sbase = static_cast<unsigned char*>(pass == 0 ? send_keys : send_pay);
      unsigned char* rbase = static_cast<unsigned char*>(pass == 0 ? recv_keys : recv_pay);
      long long at = 0;
      for (int d = 0; d < nranks; ++d) {
        sp[d] = sbase + (size_t)at * eb;
        sb[d] = (size_t)h_allB[rank].total[d] * eb;
        rp[d] = rbase + (size_t)recv_off[rank][d] * eb;
        rb[d] = (size_t)h_allB[d].total[rank] * eb;
        at += h_allB[rank].total[d];
      }
      if (sb[rank] > 0)  // my own piece stays on this GPU
        st.cuda(cudaMemcpyAsync(rp[rank], sp[rank], sb[rank], cudaMemcpyDeviceToDevice, stream));
      const int rec = prof::begin(prof::K_XCHG, stream);
      if (barrier) barrier(barrier_ctx);
      st.set(ops->exchange(ops->ctx, sp.data(), sb.data(), rp.data(), rb.data(), stream));
      if (barrier) barrier(barrier_ctx);
      prof::end(rec, stream);
    }
  }
  trace.mark("partition", stream);

  // ---- sort what I received ----
  void* result = mem.get((size_t)(n_recv > 0 ? n_recv : 1) * out_elem);
  if (result == nullptr) st.set(B2S_ERR_WORKSPACE);
  void* sort_ws = nullptr;
  if (n_recv > 0 && st.ok()) {
    size_t ws_bytes = 0;
    st.set(b2s_workspace_bytes(dtype, (size_t)n_recv, (size_t)n_recv, argsort, &ws_bytes));
    sort_ws = st.ok() ? mem.get(ws_bytes) : nullptr;
    if (st.ok() && sort_ws == nullptr) st.set(B2S_ERR_WORKSPACE);
    if (st.ok()) {
      const bool parts_ok = sender_hist && local_sort_pos32_supported((size_t)n_recv) && (size_t)n_recv < single_limit();
      if (parts_ok && (!argsort || payb == 4)) {
        // the senders counted the digits: no histogram pass over the received keys
        st.set(local_sort_received(dtype, recv_keys, argsort ? nullptr : result, argsort ? static_cast<const uint32_t*>(recv_pay) : nullptr,
                                   argsort ? static_cast<int64_t*>(result) : nullptr, (size_t)n_recv, argsort ? gmin : 0, sort_ws,
                                   ws_bytes, stream, reinterpret_cast<const unsigned int*>(recv_block), nranks));
      } else if (!argsort) {
        st.set(b2s_local_sort(dtype, recv_keys, result, nullptr, (size_t)n_recv, (size_t)n_recv, 0, 1, 1, sort_ws, ws_bytes, stream));
      } else if (payb == 4 && kb != 16 && local_sort_pos32_supported((size_t)n_recv) && (size_t)n_recv < single_limit()) {
        // the radix passes carry the 32-bit payload themselves; the last one widens it
        st.set(local_sort_payload32(dtype, recv_keys, static_cast<const uint32_t*>(recv_pay), static_cast<int64_t*>(result),
                                    (size_t)n_recv, gmin, sort_ws, ws_bytes, stream));
      } else {
        // positions inside the receive buffer first, the payload through them afterwards
        int64_t* position = static_cast<int64_t*>(mem.get((size_t)n_recv * 8));
        if (position == nullptr) st.set(B2S_ERR_WORKSPACE);
        if (st.ok())
          st.set(b2s_local_sort(dtype, recv_keys, nullptr, position, (size_t)n_recv, (size_t)n_recv, 0, 1, 1, sort_ws, ws_bytes, stream));
        if (st.ok()) {
          prof::Scope ps(prof::K_DIST, stream);
          unsigned int grid = (unsigned int)std::min<long long>((n_recv + 1023) / 1024, 148 * 16);
          if (payb == 4)
            gather_payload_kernel<uint32_t><<<grid, 256, 0, stream>>>(position, static_cast<const uint32_t*>(recv_pay), n_recv, gmin,
                                                                       static_cast<int64_t*>(result));
          else
            gather_payload_kernel<int64_t><<<grid, 256, 0, stream>>>(position, static_cast<const int64_t*>(recv_pay), n_recv, 0,
                                                                      static_cast<int64_t*>(result));
          st.cuda(cudaGetLastError());
        }
      }
    }
  }
  // temporaries are handed back only once the stream is done with them; a bounded wait that ran
  // out inside the partition kernel or the local sort shows up here
  unsigned int part_status = 0;
  st.cuda(cudaMemcpyAsync(&part_status, d_status, sizeof(part_status), cudaMemcpyDeviceToHost, stream));
  if (sort_ws != nullptr && st.ok() && dtype != B2S_COMPLEX128) st.set(b2s_check_status(sort_ws, stream));
  else st.cuda(cudaStreamSynchronize(stream));
  if (part_status != 0) st.set((int)part_status);
  trace.mark("sort(sync)");
  if (!st.ok()) return st.code;
  mem.disown(result);
  *out_ptr = result;
  *out_len = (size_t)n_recv;
  return B2S_OK;
}

// ---- N-D tiles whose sort axis is the one split over the ranks ------------------------------
// Every rank holds the same `rows` rows and a slice of each of them (extent_local elements,
// slices in rank order).  All rows at once: the rows are dealt out to the ranks, each rank
// receives the other ranks' slices of its rows (one exchange), sorts its now complete rows with
// the segmented local sort, and sends every rank its slice of the sorted rows back (a second
// exchange).  Exact extents come out by construction: no samples, no rebalancing step, and the
// cost does not depend on the number of rows.  The reference runs its sample sort over all
// segments and then shifts the results back into place (src/cupynumeric/sort/sort.cu:1351-1452,
// 1759-1773, 799-1261).
int b2s_dist_sort_nd_ops(int dtype, const void* tile_in, void* tile_out, int argsort, size_t rows, size_t extent_local,
                         const b2s_comm_ops* ops, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                         void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream)
{
  int xf       = 0;
  const int kb = kb_of(dtype, &xf);
  if (kb == 0) return B2S_ERR_UNSUPPORTED;
  if (alloc == nullptr || nranks < 1 || nranks > MAX_BUCKETS || rank < 0 || rank >= nranks) return B2S_ERR_INVALID_ARG;
  if (nranks > 1 && (ops == nullptr || ops->all_gather == nullptr || ops->exchange == nullptr)) return B2S_ERR_INVALID_ARG;
  if (rows * extent_local > 0 && (tile_in == nullptr || tile_out == nullptr)) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  Scratch mem{alloc, release, alloc_ctx, {}};
  Status st;
  const size_t out_elem = argsort ? 8 : (size_t)kb;

  // ---- everybody's extent along the sort axis, and whether everybody is in one piece ----
  std::vector<long long> all((size_t)4 * nranks);
  long long mine[4] = {(long long)extent_local, (long long)rows, 0, 0};
  long long* d_all  = static_cast<long long*>(mem.get(sizeof(long long) * 4 * (nranks + 1)));
  if (d_all == nullptr) {
    st.set(B2S_ERR_WORKSPACE);
    d_all = reinterpret_cast<long long*>(emergency_area());
    if (d_all == nullptr) return B2S_ERR_CUDA;
  }
  auto agree = [&]() -> int {
    // all-gather of (extent, rows, status): returns the first failure any rank reported
    mine[2] = st.code;
    st.cuda(cudaMemcpyAsync(d_all + 4 * nranks, mine, sizeof(mine), cudaMemcpyHostToDevice, stream));
    if (nranks > 1) {
      if (barrier) barrier(barrier_ctx);
      st.set(ops->all_gather(ops->ctx, d_all + 4 * nranks, d_all, sizeof(mine), stream));
      if (barrier) barrier(barrier_ctx);
    } else {
      st.cuda(cudaMemcpyAsync(d_all, d_all + 4, sizeof(mine), cudaMemcpyDeviceToDevice, stream));
    }
    st.cuda(cudaMemcpyAsync(all.data(), d_all, sizeof(long long) * 4 * nranks, cudaMemcpyDeviceToHost, stream));
    st.cuda(cudaStreamSynchronize(stream));
    if (!st.ok()) return st.code;
    for (int p = 0; p < nranks; ++p)
      if (all[4 * p + 2] != B2S_OK) return (int)all[4 * p + 2];
    return B2S_OK;
  };
  int rc = agree();
  if (rc != B2S_OK) return rc;
  std::vector<long long> lo(nranks + 1, 0);
  for (int p = 0; p < nranks; ++p) {
    if (all[4 * p + 1] != (long long)rows) return B2S_ERR_INVALID_ARG;  // the ranks disagree on the tile's shape
    lo[p + 1] = lo[p] + all[4 * p];
  }
  const long long extent_global = lo[nranks];
  if (rows == 0 || extent_global == 0) return B2S_OK;
  auto row_lo = [&](int q) { return (long long)rows * q / nranks; };   // rank q sorts rows [row_lo(q), row_lo(q+1))
  const long long my_rows = row_lo(rank + 1) - row_lo(rank);

  // ---- buffers: what I receive (one block per source), my complete rows, their sorted form ----
  const size_t full = (size_t)my_rows * (size_t)extent_global;
  unsigned char* stage_in  = static_cast<unsigned char*>(mem.get(full * kb + 256));
  unsigned char* full_rows = static_cast<unsigned char*>(mem.get(full * kb + 256));
  unsigned char* sorted    = static_cast<unsigned char*>(mem.get(full * out_elem + 256));
  unsigned char* stage_out = static_cast<unsigned char*>(mem.get(full * out_elem + 256));
  size_t ws_bytes = 0;
  void* sort_ws   = nullptr;
  if (full > 0) {
    st.set(b2s_workspace_bytes(dtype, full, (size_t)extent_global, argsort, &ws_bytes));
    if (st.ok()) sort_ws = mem.get(ws_bytes);
  }
  if (!stage_in || !full_rows || !sorted || !stage_out || (full > 0 && sort_ws == nullptr)) st.set(B2S_ERR_WORKSPACE);
  rc = agree();  // nobody enters the exchanges unless everybody can
  if (rc != B2S_OK) return rc;

  const unsigned char* in = static_cast<const unsigned char*>(tile_in);
  unsigned char* out      = static_cast<unsigned char*>(tile_out);
  std::vector<const void*> sp(nranks, nullptr);
  std::vector<void*> rp(nranks, nullptr);
  std::vector<size_t> sb(nranks, 0), rb(nranks, 0);
  // ---- first exchange: rank q gets rows [row_lo(q), row_lo(q+1)) of my slice, a contiguous block ----
  for (int q = 0; q < nranks; ++q) {
    const long long nq = row_lo(q + 1) - row_lo(q);
    sp[q] = in + (size_t)row_lo(q) * extent_local * kb;
    sb[q] = (size_t)nq * extent_local * kb;
    rp[q] = stage_in + (size_t)my_rows * (size_t)lo[q] * kb;   // blocks in source order
    rb[q] = (size_t)my_rows * (size_t)all[4 * q] * kb;
  }
  if (sb[rank] > 0) st.cuda(cudaMemcpyAsync(rp[rank], sp[rank], sb[rank], cudaMemcpyDeviceToDevice, stream));
  if (nranks > 1) {
    if (barrier) barrier(barrier_ctx);
    st.set(ops->exchange(ops->ctx, sp.data(), sb.data(), rp.data(), rb.data(), stream));
    if (barrier) barrier(barrier_ctx);
  }
  // the block of source q holds columns [lo[q], lo[q+1]) of my rows
  for (int q = 0; q < nranks && my_rows > 0; ++q) {
    if (all[4 * q] == 0) continue;
    st.cuda(cudaMemcpy2DAsync(full_rows + (size_t)lo[q] * kb, (size_t)extent_global * kb, rp[q], (size_t)all[4 * q] * kb,
                              (size_t)all[4 * q] * kb, (size_t)my_rows, cudaMemcpyDeviceToDevice, stream));
  }
  // ---- my rows, complete: one segmented sort; argsort positions are positions in the whole row ----
  if (full > 0 && st.ok())
    st.set(b2s_local_sort(dtype, full_rows, argsort ? nullptr : sorted, argsort ? reinterpret_cast<int64_t*>(sorted) : nullptr, full,
                          (size_t)extent_global, 0, 0, 1, sort_ws, ws_bytes, stream));
  // ---- second exchange: every rank gets its columns of my sorted rows back ----
  for (int q = 0; q < nranks; ++q) {
    const long long nq = row_lo(q + 1) - row_lo(q);
    unsigned char* block = stage_out + (size_t)my_rows * (size_t)lo[q] * out_elem;
    if (my_rows > 0 && all[4 * q] > 0)
      st.cuda(cudaMemcpy2DAsync(block, (size_t)all[4 * q] * out_elem, sorted + (size_t)lo[q] * out_elem, (size_t)extent_global * out_elem,
                                (size_t)all[4 * q] * out_elem, (size_t)my_rows, cudaMemcpyDeviceToDevice, stream));
    sp[q] = block;
    sb[q] = (size_t)my_rows * (size_t)all[4 * q] * out_elem;
    rp[q] = out + (size_t)row_lo(q) * extent_local * out_elem;   // rows sorted by rank q, my columns
    rb[q] = (size_t)nq * extent_local * out_elem;
  }
  if (sb[rank] > 0) st.cuda(cudaMemcpyAsync(rp[rank], sp[rank], sb[rank], cudaMemcpyDeviceToDevice, stream));
  if (nranks > 1) {
    if (barrier) barrier(barrier_ctx);
    st.set(ops->exchange(ops->ctx, sp.data(), sb.data(), rp.data(), rb.data(), stream));
    if (barrier) barrier(barrier_ctx);
  }
  if (sort_ws != nullptr && st.ok() && dtype != B2S_COMPLEX128) st.set(b2s_check_status(sort_ws, stream));
  else st.cuda(cudaStreamSynchronize(stream));
  return st.code;
}

// The same two calls over an NCCL communicator.
int b2s_dist_sort_1d(int dtype, const void* keys_in, size_t n_local, int64_t global_offset, int argsort,
                     void* nccl_comm, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                     void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void** out_ptr,
                     size_t* out_len, int64_t* out_global_offset, void* cuda_stream)
{
  if (nranks <= 1)
    return b2s_dist_sort_1d_ops(dtype, keys_in, n_local, global_offset, argsort, nullptr, rank, nranks, alloc, release, alloc_ctx,
                                barrier, barrier_ctx, out_ptr, out_len, out_global_offset, cuda_stream);
  if (nccl_comm == nullptr || alloc == nullptr) return B2S_ERR_INVALID_ARG;
  // the barrier's device word: from the caller's pool or, failing that, the library's own area
  void* word     = alloc(alloc_ctx, 256);
  const bool own = word != nullptr;
  if (!own) {
    unsigned char* ea = emergency_area();
    if (ea == nullptr) return B2S_ERR_CUDA;
    word = ea + EMERGENCY_BYTES - 256;
  }
  b2s_comm_ops ops{};
  int rc = b2s_nccl_comm_ops(&ops, nccl_comm, rank, nranks, word);
  if (rc == B2S_OK) {
    cudaMemsetAsync(word, 0, sizeof(int), static_cast<cudaStream_t>(cuda_stream));
    rc = b2s_dist_sort_1d_ops(dtype, keys_in, n_local, global_offset, argsort, &ops, rank, nranks, alloc, release, alloc_ctx,
                              barrier, barrier_ctx, out_ptr, out_len, out_global_offset, cuda_stream);
    b2s_nccl_comm_ops_release(&ops);
  }
  if (own && release) release(alloc_ctx, word);  // the call above synchronised the stream
  return rc;
}

int b2s_dist_rebalance_1d(size_t elem_bytes, const void* part, size_t part_len, int64_t part_global_start,
                          void* out, size_t out_len, int64_t out_global_start, void* nccl_comm, int rank,
                          int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                          b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream)
{
  if (nranks <= 1)
    return b2s_dist_rebalance_1d_ops(elem_bytes, part, part_len, part_global_start, out, out_len, out_global_start, nullptr, rank,
                                     nranks, alloc, release, alloc_ctx, barrier, barrier_ctx, cuda_stream);
  if (nccl_comm == nullptr) return B2S_ERR_INVALID_ARG;
  int word = 0;  // the exchange of the rebalance needs no barrier word
  b2s_comm_ops ops{};
  int rc = b2s_nccl_comm_ops(&ops, nccl_comm, rank, nranks, &word);
  if (rc != B2S_OK) return rc;
  rc = b2s_dist_rebalance_1d_ops(elem_bytes, part, part_len, part_global_start, out, out_len, out_global_start, &ops, rank, nranks,
                                 alloc, release, alloc_ctx, barrier, barrier_ctx, cuda_stream);
  b2s_nccl_comm_ops_release(&ops);
  return rc;
}

int b2s_dist_sort_nd(int dtype, const void* tile_in, void* tile_out, int argsort, size_t rows, size_t extent_local,
                     void* nccl_comm, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                     b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream)
{
  if (nranks <= 1)
    return b2s_dist_sort_nd_ops(dtype, tile_in, tile_out, argsort, rows, extent_local, nullptr, rank, nranks, alloc, release,
                                alloc_ctx, barrier, barrier_ctx, cuda_stream);
  if (nccl_comm == nullptr) return B2S_ERR_INVALID_ARG;
  int word = 0;  // the two exchanges need no barrier word
  b2s_comm_ops ops{};
  int rc = b2s_nccl_comm_ops(&ops, nccl_comm, rank, nranks, &word);
  if (rc != B2S_OK) return rc;
  rc = b2s_dist_sort_nd_ops(dtype, tile_in, tile_out, argsort, rows, extent_local, &ops, rank, nranks, alloc, release, alloc_ctx,
                            barrier, barrier_ctx, cuda_stream);
  b2s_nccl_comm_ops_release(&ops);
  return rc;
}
}
