// Launch counters and optional per-kernel event timing (see include/b200sort.h:
// b2s_profile_enable / b2s_profile_read / b2s_launch_count).  Process-wide; launches may be
// recorded from several host threads at once (ranks that are threads of one process).
#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/b200sort.h"
#include "b2s_prof.h"

namespace b2s {
namespace prof {

struct Rec {
  int kind;
  cudaEvent_t a, b;
};
static std::atomic<bool> g_enabled{false};
static std::mutex g_mu;                   // guards the two vectors
static std::vector<Rec> g_recs;           // event pairs in use since the last enable/reset
static std::vector<cudaEvent_t> g_pool;   // spare events
static std::atomic<unsigned long long> g_launches[K_COUNT];

static cudaEvent_t take_event()
{
  cudaEvent_t e = nullptr;
  if (!g_pool.empty()) {
    e = g_pool.back();
    g_pool.pop_back();
  } else {
    cudaEventCreate(&e);
  }
  return e;
}

static thread_local int t_account = -1;

Account::Account(int kind) : saved(t_account) { t_account = kind; }
Account::~Account() { t_account = saved; }

int begin(int kind, cudaStream_t stream)
{
  if (t_account >= 0) kind = t_account;
  ++g_launches[kind];
  if (!g_enabled.load()) return -1;
  std::lock_guard<std::mutex> lock(g_mu);
  Rec r{kind, take_event(), take_event()};
  cudaEventRecord(r.a, stream);
  g_recs.push_back(r);
  return (int)g_recs.size() - 1;
}

void end(int id, cudaStream_t stream)
{
  if (id < 0) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (id < (int)g_recs.size()) cudaEventRecord(g_recs[id].b, stream);
}

static void recycle()
{
  for (auto& r : g_recs) {
    g_pool.push_back(r.a);
    g_pool.push_back(r.b);
  }
  g_recs.clear();
}

}  // namespace prof
}  // namespace b2s

using namespace b2s::prof;

extern "C" {

int b2s_profile_enable(int on)
{
  std::lock_guard<std::mutex> lock(g_mu);
  g_enabled.store(false);
  recycle();
  // events are created here, not between the kernels that are being timed
  constexpr size_t RESERVE = 4096;
  while (on != 0 && g_pool.size() < RESERVE) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) break;
    g_pool.push_back(e);
  }
  g_enabled.store(on != 0);
  return B2S_OK;
}

int b2s_profile_read(int kind, double* total_ms, unsigned long long* launches)
{
  if (kind < 0 || kind >= K_COUNT) return B2S_ERR_INVALID_ARG;
  double tot = 0;
  unsigned long long cnt = 0;
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& r : g_recs) {
    if (r.kind != kind) continue;
    if (cudaEventSynchronize(r.b) != cudaSuccess) return B2S_ERR_CUDA;
    float ms = 0;
    if (cudaEventElapsedTime(&ms, r.a, r.b) != cudaSuccess) return B2S_ERR_CUDA;
    tot += ms;
    ++cnt;
  }
  if (total_ms) *total_ms = tot;
  if (launches) *launches = cnt;
  return B2S_OK;
}

int b2s_profile_durations(int kind, float* ms_out, size_t capacity, size_t* launches)
{
  if (kind < 0 || kind >= K_COUNT || launches == nullptr || (capacity > 0 && ms_out == nullptr)) return B2S_ERR_INVALID_ARG;
  size_t cnt = 0;
  std::lock_guard<std::mutex> lock(g_mu);
  for (auto& r : g_recs) {
    if (r.kind != kind) continue;
    if (cnt < capacity) {
      if (cudaEventSynchronize(r.b) != cudaSuccess) return B2S_ERR_CUDA;
      if (cudaEventElapsedTime(&ms_out[cnt], r.a, r.b) != cudaSuccess) return B2S_ERR_CUDA;
    }
    ++cnt;
  }
  *launches = cnt;
  return B2S_OK;
}

unsigned long long b2s_launch_count(int kind)
{
  if (kind >= 0 && kind < K_COUNT) return g_launches[kind].load();
  unsigned long long t = 0;
  for (int k = 0; k < K_COUNT; ++k) t += g_launches[k].load();
  return t;
}
}
