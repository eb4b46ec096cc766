// Peer-memory exchange of the distributed sort: every rank copies the slices it is owed straight
// out of the other ranks' sorted buffers with its own kernel (plain loads over NVLink), instead of
// pairing ncclSend/ncclRecv calls (the reference's exchange, src/cupynumeric/sort/sort.cu:1508-1745,
// goes through NCCL as well).
//
// The sorted buffers come from the caller's allocator, so they are made visible to the other
// processes with CUDA IPC handles of the allocations they sit in.  Whatever cannot be exported
// (memory that does not come from cudaMalloc, ranks living in one process) makes every rank fall
// back to the NCCL exchange: each rank's "I can" flag travels with data all ranks see.
#pragma once
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

namespace b2s {

constexpr int PEER_BUFFERS = 2;  // sorted keys, payload

// What a rank publishes about its sorted buffers (fixed size, travels with the samples).
struct PeerRecord {
  unsigned long long ok;                  // 1: the handles below can be opened
  unsigned long long pid;                 // ranks of one process cannot open each other's handles
  unsigned long long nbuf;                // buffers in use (1: keys only)
  unsigned long long off[PEER_BUFFERS];   // byte offset of the buffer inside its allocation
  cudaIpcMemHandle_t handle[PEER_BUFFERS];
  unsigned char pad_[256 - 8 * (3 + PEER_BUFFERS) - PEER_BUFFERS * sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(PeerRecord) == 256, "PeerRecord is a fixed 256-byte block");

// Base address of the allocation that holds `p` (driver entry point looked up at run time, so the
// library does not link against the driver).
inline bool allocation_base(const void* p, unsigned long long* base)
{
  typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
  static range_fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<range_fn>(f);
  }();
  if (fn == nullptr) return false;
  size_t size = 0;
  return fn(base, &size, (unsigned long long)reinterpret_cast<uintptr_t>(p)) == 0;
}

inline bool peer_exchange_enabled()
{
  const char* e = std::getenv("B2S_DIST_P2P");
  return e == nullptr || e[0] != '0';
}

// Fills `rec` for the given buffers; rec->ok stays 0 when any of them cannot be exported.
inline void export_buffers(void* const* bufs, int nbuf, PeerRecord* rec)
{
  std::memset(rec, 0, sizeof(*rec));
  rec->pid  = (unsigned long long)getpid();
  rec->nbuf = (unsigned long long)nbuf;
  if (!peer_exchange_enabled()) return;
  for (int i = 0; i < nbuf; ++i) {
    unsigned long long base = 0;
    const uintptr_t p       = reinterpret_cast<uintptr_t>(bufs[i]);
    if (bufs[i] == nullptr || (p & 255u) != 0 || !allocation_base(bufs[i], &base)) return;
    if (cudaIpcGetMemHandle(&rec->handle[i], reinterpret_cast<void*>((uintptr_t)base)) != cudaSuccess) {
      cudaGetLastError();  // not an error of the sort: the NCCL exchange takes over
      return;
    }
    rec->off[i] = (unsigned long long)p - base;
  }
  rec->ok = 1;
}

// Mappings of other processes' allocations, opened once and kept: opening costs far more than a
// sort, and allocators hand out the same blocks again and again.  A mapping keeps the other
// process's memory alive after it frees it, so the table is bounded (B2S_PEER_CACHE entries,
// 256 by default): when it is full, the mapping that has gone unused the longest and that no
// sort in flight holds is closed.
class PeerMappings {
 public:
  // Maps the allocation behind `h` (or finds it) and pins it until release(); null on failure.
  void* acquire(const cudaIpcMemHandle_t& h, std::string* key_out)
  {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::string key(reinterpret_cast<const char*>(&h), sizeof(h));
    key.push_back((char)dev);
    std::lock_guard<std::mutex> lock(mu_);
    ++clock_;
    auto it = table_.find(key);
    if (it == table_.end()) {
      if (table_.size() >= capacity()) evict_one();
      void* p = nullptr;
      if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
      }
      it = table_.emplace(key, Entry{p, 0, 0}).first;
    }
    ++it->second.users;
    it->second.last_used = clock_;
    *key_out             = key;
    return it->second.base;
  }
  void release(const std::string& key)
  {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = table_.find(key);
    if (it != table_.end() && it->second.users > 0) --it->second.users;
  }
  static PeerMappings& instance()
  {
    static PeerMappings m;
    return m;
  }

 private:
  struct Entry {
    void* base;
    int users;                     // sorts in flight that read through this mapping
    unsigned long long last_used;
  };
  static size_t capacity()
  {
    const char* e = std::getenv("B2S_PEER_CACHE");
    const long v  = e ? std::atol(e) : 256;
    return v < 1 ? 1 : (size_t)v;
  }
  void evict_one()
  {
    auto victim = table_.end();
    for (auto it = table_.begin(); it != table_.end(); ++it)
      if (it->second.users == 0 && (victim == table_.end() || it->second.last_used < victim->second.last_used))
        victim = it;
    if (victim == table_.end()) return;  // everything is in use: grow past the bound for now
    cudaIpcCloseMemHandle(victim->second.base);
    table_.erase(victim);
  }
  std::mutex mu_;
  std::map<std::string, Entry> table_;
  unsigned long long clock_ = 0;
};

// The mappings one sort holds, unpinned when the sort returns: by then its copy kernels have
// finished, because the sort synchronises its streams before it returns.
struct PeerPins {
  std::vector<std::string> keys;
  void* acquire(const cudaIpcMemHandle_t& h)
  {
    std::string k;
    void* p = PeerMappings::instance().acquire(h, &k);
    if (p != nullptr) keys.push_back(std::move(k));
    return p;
  }
  ~PeerPins()
  {
    for (const auto& k : keys) PeerMappings::instance().release(k);
  }
};

// ---- the copy kernel ----
constexpr int PULL_MAX_SEGS = 64;   // (MERGE_MAX_RUNS - 1) sources x PEER_BUFFERS
constexpr int PULL_THREADS  = 512;
constexpr int PULL_UNROLL   = 4;
constexpr unsigned long long PULL_CHUNK = (unsigned long long)PULL_THREADS * PULL_UNROLL * 4;  // 16-byte vectors

struct PullPlan {
  const uint4* src[PULL_MAX_SEGS];  // another GPU's memory, 16-byte aligned
  uint4* dst[PULL_MAX_SEGS];        // this GPU's memory, 16-byte aligned
  unsigned long long nvec[PULL_MAX_SEGS];
  int nseg;
  int ctas_per_seg;
};

__device__ __forceinline__ uint4 load_peer(const uint4* p)
{
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// CTA b works on segment b % nseg, so that at any time every source GPU is being read by some
// CTAs of every destination: no source's links carry the whole exchange alone.
static __global__ void __launch_bounds__(PULL_THREADS) pull_kernel(const __grid_constant__ PullPlan plan)
{
  const int seg                  = (int)(blockIdx.x % (unsigned int)plan.nseg);
  const unsigned long long first = blockIdx.x / (unsigned int)plan.nseg;
  const uint4* s                 = plan.src[seg];
  uint4* d                       = plan.dst[seg];
  const unsigned long long nv    = plan.nvec[seg];
  for (unsigned long long c0 = first * PULL_CHUNK; c0 < nv; c0 += (unsigned long long)plan.ctas_per_seg * PULL_CHUNK) {
    const unsigned long long c1 = c0 + PULL_CHUNK < nv ? c0 + PULL_CHUNK : nv;
    for (unsigned long long v = c0 + threadIdx.x; v < c1; v += (unsigned long long)PULL_THREADS * PULL_UNROLL) {
      uint4 r[PULL_UNROLL];
#pragma unroll
      for (int u = 0; u < PULL_UNROLL; ++u) {
        const unsigned long long vv = v + (unsigned long long)u * PULL_THREADS;
        if (vv < c1) r[u] = load_peer(s + vv);
      }
#pragma unroll
      for (int u = 0; u < PULL_UNROLL; ++u) {
        const unsigned long long vv = v + (unsigned long long)u * PULL_THREADS;
        if (vv < c1) d[vv] = r[u];
      }
    }
  }
}

}  // namespace b2s
