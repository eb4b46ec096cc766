// Distributed 1-D sort over the GPUs of one NVSwitch box: local sort -> regular oversampling ->
// NCCL all-gather of samples -> splitters -> cut positions -> NCCL all-gather of counts ->
// one grouped send/recv exchange of keys (and indices) -> stable k-way merge.
// Replaces sample_sort_nccl_nd for 1-D arrays (src/cupynumeric/sort/sort.cu:1270-1784) and the
// surrounding buffer handling of SortImplBody<GPU> (sort.cu:1797-1940).
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <vector>

#include "../../include/b200sort.h"
#include "b2s_common.cuh"
#include "b2s_peer.cuh"

namespace b2s {
// defined with the local sort
bool local_sort_pos32_supported(size_t n);
int local_sort_pos32(int dtype, const void* keys_in, void* keys_out, uint32_t* pos_out, size_t n, void* ws,
                     size_t ws_bytes, cudaStream_t stream);
}  // namespace b2s
#include "b2s_dist_host.h"
#include "b2s_merge.cuh"
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
    default: return 0;
  }
}

// Regular samples of the locally sorted keys, as (ordered key, rank, position) triples.
template <int KB>
__global__ void sample_kernel(const void* sorted, long long n, int s, int rank, int xf, Sample* out)
{
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= s) return;
  Sample sm;
  const long long s_eff = n < s ? n : s;
  if (j < s_eff) {
    const long long p = sample_position(j, s_eff, n);
    sm.okey  = okey_at<KB>(sorted, p, xf);
    sm.pos   = p;
    sm.rank  = rank;
    sm.valid = 1;
  } else {
    sm.okey = ~0ull;
    sm.pos = 0;
    sm.rank = rank;
    sm.valid = 0;
  }
  out[j] = sm;
}

// cuts[k] for k = 1..nranks-1: how many of my sorted elements go to ranks < k.
template <int KB>
__global__ void cut_kernel(const void* sorted, long long n, const Sample* splitters, int nranks, int rank,
                           int xf, long long* cuts, long long tag0, long long tag1, long long tag2)
{
  const int k = blockIdx.x * blockDim.x + threadIdx.x + 1;
  if (k >= nranks) return;
  const Sample sp = splitters[k - 1];
  long long c;
  if (!sp.valid) {
    c = n;  // no populated sample anywhere right of this splitter
  } else {
    const long long lower = lower_bound_okey<KB>(sorted, 0, n, sp.okey, xf);
    const long long upper = sp.okey == ~0ull ? n : lower_bound_okey<KB>(sorted, lower, n, sp.okey + 1, xf);
    c = cut_position(sp, rank, lower, upper);
  }
  cuts[k] = c;
  if (k == 1) {
    cuts[0]          = 0;
    cuts[nranks]     = n;
    cuts[nranks + 1] = tag0;  // three words that travel with the cuts to every rank
    cuts[nranks + 2] = tag1;
    cuts[nranks + 3] = tag2;
  }
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

// Phases of the exchange/merge pipeline.
#ifndef B2S_DIST_PHASES
#define B2S_DIST_PHASES 2
#endif
constexpr int DIST_PHASES = B2S_DIST_PHASES;

// One extra stream per device for the exchange, created on first use and kept.
static cudaStream_t exchange_stream()
{
  static cudaStream_t streams[64] = {};
  static std::mutex mu;  // two host threads may ask for the same device's stream together
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (streams[dev] == nullptr) {
    if (cudaStreamCreateWithFlags(&streams[dev], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
  }
  return streams[dev];
}

// Host-side phase trace of the distributed sort (B2S_DIST_TRACE=1, rank 0 prints).
struct PhaseTrace {
  bool on;
  std::chrono::steady_clock::time_point t0;
  char line[512] = {0};
  int used = 0;
  int rk = 0;
  explicit PhaseTrace(int rank) : on(std::getenv("B2S_DIST_TRACE") != nullptr && (rank == 0 || std::getenv("B2S_DIST_TRACE")[0] == 'a')), rk(rank), t0(std::chrono::steady_clock::now()) {}
  void mark(const char* what)
  {
    if (!on) return;
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

// CUDA events that are destroyed on every way out of the function that owns them
struct Events {
  std::vector<cudaEvent_t> ev;
  cudaEvent_t make()
  {
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    ev.push_back(e);
    return e;
  }
  ~Events()
  {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
};

#define CK_CUDA(x) do { if ((x) != cudaSuccess) return B2S_ERR_CUDA; } while (0)
#define CK_NCCL(x) do { if ((x) != ncclSuccess) return B2S_ERR_NCCL; } while (0)

}  // namespace b2s

using namespace b2s;

extern "C" {

void b2s_host_sort_samples(void* samples, size_t count)
{
  Sample* s = static_cast<Sample*>(samples);
  std::sort(s, s + count, [](const Sample& a, const Sample& b) { return sample_less(a, b); });
}

int b2s_host_select_splitters(void* samples, size_t count, int nranks, void* splitters_out)
{
  if (samples == nullptr || splitters_out == nullptr || nranks < 1) return B2S_ERR_INVALID_ARG;
  Sample* s   = static_cast<Sample*>(samples);
  Sample* out = static_cast<Sample*>(splitters_out);
  b2s_host_sort_samples(s, count);
  long long populated = 0;
  while ((size_t)populated < count && s[populated].valid) ++populated;
  for (int k = 1; k < nranks; ++k) {
    if (populated == 0) {
      out[k - 1] = Sample{~0ull, 0, 0, 0};
    } else {
      out[k - 1] = s[splitter_index(k, populated, nranks)];
    }
  }
  return B2S_OK;
}

long long b2s_host_sample_position(long long j, long long s, long long n) { return sample_position(j, s, n); }

long long b2s_host_cut_position(const void* splitter, int my_rank, long long lower, long long upper)
{
  return cut_position(*static_cast<const Sample*>(splitter), my_rank, lower, upper);
}

int b2s_samples_per_rank(void) { return SAMPLES_PER_RANK; }

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
  if (kb == 0) return B2S_ERR_UNSUPPORTED;
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

int b2s_dist_rebalance_1d(size_t elem_bytes, const void* part, size_t part_len, int64_t part_global_start,
                          void* out, size_t out_len, int64_t out_global_start, void* nccl_comm, int rank,
                          int nranks, b2s_alloc_fn alloc, b2s_free_fn release, void* alloc_ctx,
                          b2s_barrier_fn barrier, void* barrier_ctx, void* cuda_stream)
{
  if (elem_bytes == 0 || nranks < 1 || rank < 0 || rank >= nranks || alloc == nullptr) return B2S_ERR_INVALID_ARG;
  if ((part_len > 0 && part == nullptr) || (out_len > 0 && out == nullptr)) return B2S_ERR_INVALID_ARG;
  if (nranks > 1 && nccl_comm == nullptr) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  ncclComm_t comm     = static_cast<ncclComm_t>(nccl_comm);
  Scratch mem{alloc, release, alloc_ctx, {}};
  // every rank learns where every rank's sorted part and output extent lie in the global order
  long long mine[4] = {(long long)part_global_start, (long long)part_len, (long long)out_global_start, (long long)out_len};
  std::vector<long long> all((size_t)4 * nranks);
  if (nranks == 1) {
    std::copy(mine, mine + 4, all.begin());
  } else {
    long long* d_all = static_cast<long long*>(mem.get(sizeof(long long) * 4 * (nranks + 1)));
    if (d_all == nullptr) return B2S_ERR_WORKSPACE;
    CK_CUDA(cudaMemcpyAsync(d_all + 4 * nranks, mine, sizeof(mine), cudaMemcpyHostToDevice, stream));
    if (barrier) barrier(barrier_ctx);
    CK_NCCL(ncclAllGather(d_all + 4 * nranks, d_all, sizeof(mine), ncclUint8, comm, stream));
    if (barrier) barrier(barrier_ctx);
    CK_CUDA(cudaMemcpyAsync(all.data(), d_all, sizeof(long long) * 4 * nranks, cudaMemcpyDeviceToHost, stream));
    CK_CUDA(cudaStreamSynchronize(stream));
  }
  long long parts_total = 0, outs_total = 0;
  for (int p = 0; p < nranks; ++p) {
    parts_total += all[4 * p + 1];
    outs_total += all[4 * p + 3];
  }
  if (parts_total != outs_total) return B2S_ERR_INVALID_ARG;  // extents must tile what was sorted
  const unsigned char* src = static_cast<const unsigned char*>(part);
  unsigned char* dst       = static_cast<unsigned char*>(out);
  auto overlap = [](long long a0, long long a1, long long b0, long long b1, long long* lo, long long* hi) {
    *lo = a0 > b0 ? a0 : b0;
    *hi = a1 < b1 ? a1 : b1;
    return *hi > *lo;
  };
  const long long ps = mine[0], pe = mine[0] + mine[1], os = mine[2], oe = mine[2] + mine[3];
  if (barrier) barrier(barrier_ctx);
  if (nranks > 1) CK_NCCL(ncclGroupStart());
  for (int i = 1; i < nranks; ++i) {
    const int to = (rank + i) % nranks, from = (rank - i + nranks) % nranks;
    long long lo, hi;
    if (overlap(ps, pe, all[4 * to + 2], all[4 * to + 2] + all[4 * to + 3], &lo, &hi))
      CK_NCCL(ncclSend(src + (size_t)(lo - ps) * elem_bytes, (size_t)(hi - lo) * elem_bytes, ncclUint8, to, comm, stream));
    if (overlap(all[4 * from], all[4 * from] + all[4 * from + 1], os, oe, &lo, &hi))
      CK_NCCL(ncclRecv(dst + (size_t)(lo - os) * elem_bytes, (size_t)(hi - lo) * elem_bytes, ncclUint8, from, comm, stream));
  }
  if (nranks > 1) CK_NCCL(ncclGroupEnd());
  if (barrier) barrier(barrier_ctx);
  long long lo, hi;
  if (overlap(ps, pe, os, oe, &lo, &hi))
    CK_CUDA(cudaMemcpyAsync(dst + (size_t)(lo - os) * elem_bytes, src + (size_t)(lo - ps) * elem_bytes,
                            (size_t)(hi - lo) * elem_bytes, cudaMemcpyDeviceToDevice, stream));
  CK_CUDA(cudaStreamSynchronize(stream));
  return B2S_OK;
}

int b2s_nccl_unique_id(void* out128)
{
  static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
  if (out128 == nullptr) return B2S_ERR_INVALID_ARG;
  CK_NCCL(ncclGetUniqueId(static_cast<ncclUniqueId*>(out128)));
  return B2S_OK;
}

int b2s_nccl_comm_create(void** comm, int nranks, const void* id128, int rank)
{
  if (comm == nullptr || id128 == nullptr) return B2S_ERR_INVALID_ARG;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclComm_t c;
  CK_NCCL(ncclCommInitRank(&c, nranks, id, rank));
  *comm = c;
  return B2S_OK;
}

int b2s_nccl_comm_destroy(void* comm)
{
  if (comm == nullptr) return B2S_OK;
  CK_NCCL(ncclCommDestroy(static_cast<ncclComm_t>(comm)));
  return B2S_OK;
}

int b2s_dist_sort_1d(int dtype, const void* keys_in, size_t n_local, int64_t global_offset, int argsort,
                     void* nccl_comm, int rank, int nranks, b2s_alloc_fn alloc, b2s_free_fn release,
                     void* alloc_ctx, b2s_barrier_fn barrier, void* barrier_ctx, void** out_ptr,
                     size_t* out_len, int64_t* out_global_offset, void* cuda_stream)
{
  int xf       = 0;
  const int kb = kb_of(dtype, &xf);
  if (kb == 0) return B2S_ERR_UNSUPPORTED;
  if (alloc == nullptr || out_ptr == nullptr || out_len == nullptr || nranks < 1 || rank < 0 || rank >= nranks)
    return B2S_ERR_INVALID_ARG;
  if (nranks > MERGE_MAX_RUNS) return B2S_ERR_UNSUPPORTED;
  if (nranks > 1 && nccl_comm == nullptr) return B2S_ERR_INVALID_ARG;
  if (n_local > 0 && keys_in == nullptr) return B2S_ERR_INVALID_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  ncclComm_t comm     = static_cast<ncclComm_t>(nccl_comm);
  Scratch mem{alloc, release, alloc_ctx, {}};
  const long long n = (long long)n_local;
  PhaseTrace trace(rank);
  int local_status = B2S_OK;

  // ---- 1. local sort; indices are global positions (sort.cu:1851-1854) ----
  // With more than one rank an argsort carries 32-bit local positions through the exchange where
  // the local sort can produce them; the merge adds the source rank's offset.  Each rank tells
  // the others which form it sends (payload width and offset travel with the cut positions).
  const bool pos32 = argsort && nranks > 1 && local_sort_pos32_supported(n_local);
  const size_t pb  = pos32 ? 4 : 8;  // bytes per payload element I send
  // 16 spare bytes: the peer-memory exchange copies whole 16-byte vectors out of these buffers
  void* keys       = mem.get((size_t)n * kb + 16);
  unsigned char* idx = argsort ? static_cast<unsigned char*>(mem.get((size_t)n * pb + 16)) : nullptr;
  if (keys == nullptr || (argsort && idx == nullptr)) return B2S_ERR_WORKSPACE;
  void* sort_ws = nullptr;
  if (n > 0) {
    size_t ws_bytes = 0;
    int rc = b2s_workspace_bytes(dtype, n_local, n_local, argsort, &ws_bytes);
    if (rc != B2S_OK) return rc;
    void* ws = mem.get(ws_bytes);
    if (ws == nullptr) return B2S_ERR_WORKSPACE;
    sort_ws = ws;
    if (pos32)
      rc = local_sort_pos32(dtype, keys_in, keys, reinterpret_cast<uint32_t*>(idx), n_local, ws, ws_bytes, stream);
    else
      rc = b2s_local_sort(dtype, keys_in, keys, reinterpret_cast<int64_t*>(idx), n_local, n_local, global_offset, 1, 1,
                          ws, ws_bytes, stream);
    if (rc != B2S_OK) return rc;
    if (nranks == 1) {
      rc = b2s_check_status(ws, stream);
      if (rc != B2S_OK) return rc;
    }
    // the workspace is released after the exchange below has synchronised the stream
    if (nranks == 1) mem.drop(ws);
  }
  if (nranks == 1) {
    void* result = argsort ? static_cast<void*>(idx) : keys;  // one rank: idx holds int64 global indices
    mem.disown(result);
    *out_ptr = result;
    *out_len = n_local;
    if (out_global_offset) *out_global_offset = 0;
    return B2S_OK;
  }

  trace.mark("enqueue_local_sort");
  // ---- 2. samples: all-gather, order on the host, pick the splitters ----
  // Each destination's value range is cut once more into PH consecutive sub-ranges ("phases"):
  // while the runs of phase k are being merged, NCCL already moves the runs of phase k+1.
  const int nph      = DIST_PHASES;  // the same on every rank by construction
  const int nb       = nranks * nph;  // buckets: bucket q goes to rank q / nph in phase q % nph
  const int s        = SAMPLES_PER_RANK;
  // every rank's block of the first all-gather: its samples, then what the others need to read
  // its sorted buffers directly (PeerRecord)
  const size_t blk      = sizeof(Sample) * s + sizeof(PeerRecord);
  unsigned char* d_blk  = static_cast<unsigned char*>(mem.get(blk * nranks));
  Sample* d_split    = static_cast<Sample*>(mem.get(sizeof(Sample) * nb));
  long long* d_cuts  = static_cast<long long*>(mem.get(sizeof(long long) * (nb + 4)));
  long long* d_count = static_cast<long long*>(mem.get(sizeof(long long) * nranks * (nb + 4)));
  int* d_done        = static_cast<int*>(mem.get(256));
  if (!d_blk || !d_split || !d_cuts || !d_count || !d_done) return B2S_ERR_WORKSPACE;
  PeerRecord my_rec;
  {
    void* bufs[PEER_BUFFERS] = {keys, idx};
    export_buffers(bufs, argsort ? 2 : 1, &my_rec);
  }
  {
    prof::Scope ps(prof::K_DIST, stream);
    by_width(kb, [&](auto w) {
      sample_kernel<decltype(w)::value><<<(s + 127) / 128, 128, 0, stream>>>(
        keys, n, s, rank, xf, reinterpret_cast<Sample*>(d_blk + (size_t)rank * blk));
      return cudaSuccess;
    });
  }
  CK_CUDA(cudaGetLastError());
  CK_CUDA(cudaMemcpyAsync(d_blk + (size_t)rank * blk + sizeof(Sample) * s, &my_rec, sizeof(PeerRecord),
                          cudaMemcpyHostToDevice, stream));
  if (barrier) barrier(barrier_ctx);
  CK_NCCL(ncclAllGather(d_blk + (size_t)rank * blk, d_blk, blk, ncclUint8, comm, stream));
  if (barrier) barrier(barrier_ctx);
  std::vector<unsigned char> h_blk(blk * nranks);
  std::vector<Sample> h_samples((size_t)s * nranks), h_split(nb);
  CK_CUDA(cudaMemcpyAsync(h_blk.data(), d_blk, blk * nranks, cudaMemcpyDeviceToHost, stream));
  CK_CUDA(cudaStreamSynchronize(stream));
  std::vector<PeerRecord> recs(nranks);
  for (int p = 0; p < nranks; ++p) {
    std::memcpy(&h_samples[(size_t)p * s], &h_blk[(size_t)p * blk], sizeof(Sample) * s);
    std::memcpy(&recs[p], &h_blk[(size_t)p * blk + sizeof(Sample) * s], sizeof(PeerRecord));
  }
  // Can I read everybody's buffers?  All ranks see the same records, so they agree on the first
  // part; whether the mappings open is local and travels with the cut positions below.
  std::vector<const unsigned char*> peer_keys(nranks, nullptr), peer_idx(nranks, nullptr);
  PeerPins pins;  // declared after `mem` and before any kernel that reads a peer is launched
  long long can_pull = 1;
  for (int p = 0; p < nranks && can_pull; ++p) {
    if (!recs[p].ok || recs[p].nbuf != (unsigned long long)(argsort ? 2 : 1)) can_pull = 0;
    if (p != rank && recs[p].pid == my_rec.pid) can_pull = 0;
  }
  for (int p = 0; p < nranks && can_pull; ++p) {
    if (p == rank) continue;
    const unsigned char* kbase = static_cast<const unsigned char*>(pins.acquire(recs[p].handle[0]));
    const unsigned char* ibase = argsort ? static_cast<const unsigned char*>(pins.acquire(recs[p].handle[1])) : nullptr;
    if (kbase == nullptr || (argsort && ibase == nullptr)) {
      can_pull = 0;
      break;
    }
    peer_keys[p] = kbase + recs[p].off[0];
    peer_idx[p]  = argsort ? ibase + recs[p].off[1] : nullptr;
  }
  trace.mark("local_sort+samples(sync)");
  if (sort_ws != nullptr) {
    // a wait inside the local sort that ran out shows up here; every rank still goes on to the
    // collectives below so that nobody is left waiting, and the error is returned at the end
    const int st = b2s_check_status(sort_ws, stream);
    if (st != B2S_OK) local_status = st;
  }
  b2s_host_select_splitters(h_samples.data(), h_samples.size(), nb, h_split.data());
  CK_CUDA(cudaMemcpyAsync(d_split, h_split.data(), sizeof(Sample) * (nb - 1), cudaMemcpyHostToDevice, stream));

  // ---- 3. where the splitters cut my data; every rank learns every rank's cut positions ----
  {
    prof::Scope ps(prof::K_DIST, stream);
    by_width(kb, [&](auto w) {
      cut_kernel<decltype(w)::value><<<(nb + 63) / 64, 64, 0, stream>>>(keys, n, d_split, nb, rank, xf, d_cuts,
                                                                        (long long)pb, (long long)global_offset, can_pull);
      return cudaSuccess;
    });
  }
  CK_CUDA(cudaGetLastError());
  const size_t row = (size_t)nb + 4;  // nb + 1 cut positions, payload width, global offset, can-pull flag
  std::vector<long long> h_allcuts((size_t)nranks * row);
  if (barrier) barrier(barrier_ctx);
  CK_NCCL(ncclAllGather(d_cuts, d_count, sizeof(long long) * row, ncclUint8, comm, stream));
  if (barrier) barrier(barrier_ctx);
  CK_CUDA(cudaMemcpyAsync(h_allcuts.data(), d_count, sizeof(long long) * nranks * row, cudaMemcpyDeviceToHost, stream));
  CK_CUDA(cudaStreamSynchronize(stream));
  trace.mark("cuts+counts(sync)");
  for (int src = 0; src < nranks; ++src)
    for (int q = 0; q < nb; ++q)
      if (h_allcuts[src * row + q] > h_allcuts[src * row + q + 1]) return B2S_ERR_INVALID_ARG;  // protocol mismatch
  bool use_pull = true;  // the same on every rank: everybody sees everybody's flag
  for (int src = 0; src < nranks; ++src) use_pull = use_pull && h_allcuts[src * row + nb + 3] == 1;
  std::vector<size_t> pay_bytes(nranks);
  for (int src = 0; src < nranks; ++src) {
    const long long w = h_allcuts[src * row + nb + 1];
    if (w != 4 && w != 8) return B2S_ERR_INVALID_ARG;
    pay_bytes[src] = (size_t)w;
  }
  const long long* my_cuts = &h_allcuts[(size_t)rank * row];

  // ---- 4. exchange and merge, phase by phase ----
  // My slice [cuts[q], cuts[q+1]) of bucket q goes to rank q / nph.  A slice starts wherever its
  // splitter cut the sorted data, usually not on a 16-byte boundary, and NCCL's copies are much
  // slower from unaligned addresses: each transfer starts at the slice's start rounded down to
  // XFER_ALIGN elements and the receiver, who knows the sender's cut positions, skips the
  // leading elements.  Runs land on aligned offsets of the receive buffer.
  constexpr long long XFER_ALIGN = 32;
  std::vector<MergeRuns> runs(nph);
  std::vector<std::vector<long long>> recv_off(nph, std::vector<long long>(nranks)), lead(nph, std::vector<long long>(nranks));
  std::vector<long long> ph_total(nph, 0);
  long long total = 0, slots = 0;
  for (int ph = 0; ph < nph; ++ph) {
    runs[ph]       = MergeRuns{};
    runs[ph].nruns = nranks;
    const int q    = rank * nph + ph;
    for (int p = 0; p < nranks; ++p) {
      const long long start = h_allcuts[p * row + q], end = h_allcuts[p * row + q + 1];
      runs[ph].len[p] = end - start;
      lead[ph][p]     = p == rank ? 0 : start % XFER_ALIGN;
      recv_off[ph][p] = slots;
      slots += (lead[ph][p] + runs[ph].len[p] + XFER_ALIGN - 1) / XFER_ALIGN * XFER_ALIGN;
      ph_total[ph] += runs[ph].len[p];
    }
    total += ph_total[ph];
  }
  unsigned char* r_keys = static_cast<unsigned char*>(mem.get((size_t)slots * kb));
  unsigned char* r_idx  = argsort ? static_cast<unsigned char*>(mem.get((size_t)slots * 8)) : nullptr;
  void* result          = mem.get((size_t)total * (argsort ? 8 : kb));
  if (r_keys == nullptr || (argsort && r_idx == nullptr) || result == nullptr) return B2S_ERR_WORKSPACE;
  std::vector<void*> tcuts(nph, nullptr);
  for (int ph = 0; ph < nph; ++ph) {
    for (int p = 0; p < nranks; ++p) {
      runs[ph].keys[p] = r_keys + (size_t)(recv_off[ph][p] + lead[ph][p]) * kb;
      // a run's payload sits at the same element offset as its keys, whatever its width
      runs[ph].idx[p]      = argsort ? r_idx + (size_t)recv_off[ph][p] * 8 + (size_t)lead[ph][p] * pay_bytes[p] : nullptr;
      runs[ph].idx_bytes[p] = (int)pay_bytes[p];
      runs[ph].idx_base[p]  = pay_bytes[p] == 4 ? h_allcuts[p * row + nb + 2] : 0;
    }
    if (ph_total[ph] > 0) {
      size_t mws = 0;
      b2s_kway_merge_workspace_bytes((size_t)ph_total[ph], nranks, &mws);
      tcuts[ph] = mem.get(mws);
      if (tcuts[ph] == nullptr) return B2S_ERR_WORKSPACE;
    }
  }
  const unsigned char* k_bytes = static_cast<const unsigned char*>(keys);
  trace.mark("alloc_recv");

  // The exchange runs on a stream of its own so that it overlaps the merges on the caller's.
  cudaStream_t xs = exchange_stream();
  if (xs == nullptr) return B2S_ERR_CUDA;
  Events events;
  cudaEvent_t ev_ready = events.make();
  std::vector<cudaEvent_t> ev_done(nph, nullptr);
  for (auto& e : ev_done) e = events.make();
  if (ev_ready == nullptr) return B2S_ERR_CUDA;
  for (auto e : ev_done)
    if (e == nullptr) return B2S_ERR_CUDA;
  CK_CUDA(cudaEventRecord(ev_ready, stream));
  CK_CUDA(cudaStreamWaitEvent(xs, ev_ready, 0));
  for (int ph = 0; ph < nph && use_pull; ++ph) {
    // One kernel copies this phase's slices out of the other ranks' sorted buffers.  Their
    // contents are final: the all-gather of the cut positions above completed after every
    // rank's local sort in stream order.
    PullPlan plan{};
    for (int i = 1; i < nranks; ++i) {
      const int from = (rank + i) % nranks;
      if (runs[ph].len[from] <= 0) continue;
      const long long start = h_allcuts[from * row + (size_t)rank * nph + ph];  // their slice for me
      const long long a0    = start - lead[ph][from];
      const size_t cnt      = (size_t)(lead[ph][from] + runs[ph].len[from]);
      plan.src[plan.nseg]   = reinterpret_cast<const uint4*>(peer_keys[from] + (size_t)a0 * kb);
      plan.dst[plan.nseg]   = reinterpret_cast<uint4*>(r_keys + (size_t)recv_off[ph][from] * kb);
      plan.nvec[plan.nseg]  = (cnt * kb + 15) / 16;
      ++plan.nseg;
      if (argsort) {
        plan.src[plan.nseg]  = reinterpret_cast<const uint4*>(peer_idx[from] + (size_t)a0 * pay_bytes[from]);
        plan.dst[plan.nseg]  = reinterpret_cast<uint4*>(r_idx + (size_t)recv_off[ph][from] * 8);
        plan.nvec[plan.nseg] = (cnt * pay_bytes[from] + 15) / 16;
        ++plan.nseg;
      }
    }
    if (plan.nseg > 0) {
      for (int i = 0; i < plan.nseg; ++i)
        if (((reinterpret_cast<uintptr_t>(plan.src[i]) | reinterpret_cast<uintptr_t>(plan.dst[i])) & 15u) != 0)
          return B2S_ERR_INVALID_ARG;  // cannot happen with 256-byte aligned buffers and 32-element starts
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      plan.ctas_per_seg = (2 * sms + plan.nseg - 1) / plan.nseg;
      prof::begin(prof::K_XCHG, xs);
      pull_kernel<<<(unsigned int)(plan.nseg * plan.ctas_per_seg), PULL_THREADS, 0, xs>>>(plan);
      prof::end(prof::K_XCHG, xs);
      CK_CUDA(cudaGetLastError());
    }
    CK_CUDA(cudaEventRecord(ev_done[ph], xs));
  }
  if (use_pull) {
    // nobody may release or reuse its sorted buffers before every rank has finished reading
    // them: a collective behind the copy kernels, which the final synchronisation waits for
    CK_CUDA(cudaMemsetAsync(d_done, 0, sizeof(int), xs));
    if (barrier) barrier(barrier_ctx);
    CK_NCCL(ncclAllReduce(d_done, d_done, 1, ncclInt32, ncclSum, comm, xs));
    if (barrier) barrier(barrier_ctx);
  }
  for (int ph = 0; ph < nph && !use_pull; ++ph) {
    if (barrier) barrier(barrier_ctx);
    prof::begin(prof::K_XCHG, xs);
    CK_NCCL(ncclGroupStart());
    for (int i = 1; i < nranks; ++i) {
      const int to = (rank + i) % nranks, from = (rank - i + nranks) % nranks;
      const long long c0 = my_cuts[to * nph + ph], c1 = my_cuts[to * nph + ph + 1];
      if (c1 > c0) {
        const long long a0 = c0 - c0 % XFER_ALIGN;
        const size_t cnt   = (size_t)(c1 - a0);
        CK_NCCL(ncclSend(k_bytes + (size_t)a0 * kb, cnt * kb, ncclUint8, to, comm, xs));
        if (argsort) CK_NCCL(ncclSend(idx + (size_t)a0 * pb, cnt * pb, ncclUint8, to, comm, xs));
      }
      if (runs[ph].len[from] > 0) {
        const size_t cnt = (size_t)(lead[ph][from] + runs[ph].len[from]);
        CK_NCCL(ncclRecv(r_keys + (size_t)recv_off[ph][from] * kb, cnt * kb, ncclUint8, from, comm, xs));
        if (argsort)
          CK_NCCL(ncclRecv(r_idx + (size_t)recv_off[ph][from] * 8, cnt * pay_bytes[from], ncclUint8, from, comm, xs));
      }
    }
    CK_NCCL(ncclGroupEnd());
    prof::end(prof::K_XCHG, xs);
    if (barrier) barrier(barrier_ctx);
    CK_CUDA(cudaEventRecord(ev_done[ph], xs));
  }
  trace.mark("enqueue_exchange");

  // ---- 5. per phase: my own slice, then the stable k-way merge in rank order ----
  long long out_off = 0;
  for (int ph = 0; ph < nph; ++ph) {
    const long long c0 = my_cuts[rank * nph + ph], c1 = my_cuts[rank * nph + ph + 1];
    if (c1 > c0) {  // my own slice stays on this GPU
      CK_CUDA(cudaMemcpyAsync(r_keys + (size_t)recv_off[ph][rank] * kb, k_bytes + (size_t)c0 * kb,
                              (size_t)(c1 - c0) * kb, cudaMemcpyDeviceToDevice, stream));
      if (argsort)
        CK_CUDA(cudaMemcpyAsync(r_idx + (size_t)recv_off[ph][rank] * 8, idx + (size_t)c0 * pb, (size_t)(c1 - c0) * pb,
                                cudaMemcpyDeviceToDevice, stream));
    }
    CK_CUDA(cudaStreamWaitEvent(stream, ev_done[ph], 0));
    if (ph_total[ph] > 0) {
      void* dst = static_cast<unsigned char*>(result) + (size_t)out_off * (argsort ? 8 : kb);
      int rc    = merge_runs(kb, xf, runs[ph], ph_total[ph], argsort != 0, dst, static_cast<long long*>(tcuts[ph]), stream);
      if (rc != B2S_OK) return rc;
    }
    out_off += ph_total[ph];
  }
  trace.mark("enqueue_merge");
  // temporaries are handed back only once the stream is done with them
  CK_CUDA(cudaStreamSynchronize(stream));
  CK_CUDA(cudaStreamSynchronize(xs));
  trace.mark("exchange+merge(sync)");
  mem.disown(result);
  *out_ptr = result;
  *out_len = (size_t)total;
  if (out_global_offset) {
    long long before = 0;  // elements that end up on lower ranks
    for (int d = 0; d < rank; ++d)
      for (int src = 0; src < nranks; ++src)
        before += h_allcuts[src * row + (size_t)(d + 1) * nph] - h_allcuts[src * row + (size_t)d * nph];
    *out_global_offset = before;
  }
  return local_status;
}
}
