// Peer-memory side of the distributed sort: every rank writes the elements it owes another rank
// straight into that rank's receive buffer with plain stores over NVLink, inside the kernel that
// partitions its tile (the reference packs, then pairs ncclSend/ncclRecv calls,
// src/cupynumeric/sort/sort.cu:1508-1745).
//
// The receive buffers come from the caller's allocator.  Ranks that are processes of their own see
// each other's buffers through CUDA IPC handles of the allocations they sit in; ranks that share
// a process use the addresses directly.  Whatever cannot be reached (memory that does not come
// from cudaMalloc, devices without peer access) makes every rank fall back to the collective
// exchange of the b2s_comm_ops table: each rank's "I can" flag travels with data all ranks see.
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

// What a rank publishes about its receive buffers (fixed size, travels with the samples).
struct PeerRecord {
  unsigned long long ok;                  // 1: the handles below can be opened
  unsigned long long pid;                 // ranks of one process use `ptr` instead of the handles
  unsigned long long nbuf;                // buffers in use (1: keys only)
  unsigned long long device;              // CUDA device ordinal inside the owner's process
  unsigned long long ptr[PEER_BUFFERS];   // the buffer's address in the owner's process
  unsigned long long off[PEER_BUFFERS];   // byte offset of the buffer inside its allocation
  cudaIpcMemHandle_t handle[PEER_BUFFERS];
  unsigned char pad_[256 - 8 * (4 + 2 * PEER_BUFFERS) - PEER_BUFFERS * sizeof(cudaIpcMemHandle_t)];
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
  int dev   = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  rec->device = (unsigned long long)dev;
  if (!peer_exchange_enabled()) return;
  for (int i = 0; i < nbuf; ++i) {
    unsigned long long base = 0;
    const uintptr_t p       = reinterpret_cast<uintptr_t>(bufs[i]);
    if (bufs[i] == nullptr || (p & 255u) != 0) return;
    rec->ptr[i] = (unsigned long long)p;
    if (!allocation_base(bufs[i], &base)) return;
    if (cudaIpcGetMemHandle(&rec->handle[i], reinterpret_cast<void*>((uintptr_t)base)) != cudaSuccess) {
      cudaGetLastError();  // not an error of the sort: the collective exchange takes over
      return;
    }
    rec->off[i] = (unsigned long long)p - base;
  }
  rec->ok = 1;
}

// A buffer of a rank that lives in this process, on device `their_dev`: usable as it is on the
// same device, after enabling peer access on another one.
inline bool same_process_reachable(int their_dev)
{
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (dev == their_dev) return true;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, dev, their_dev) != cudaSuccess || !can) return false;
  const cudaError_t e = cudaDeviceEnablePeerAccess(their_dev, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
  return e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled;
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

// The mappings one sort holds, unpinned when the sort returns: by then every kernel that wrote
// through them has finished, because the sort synchronises its stream before it returns.
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

}  // namespace b2s
