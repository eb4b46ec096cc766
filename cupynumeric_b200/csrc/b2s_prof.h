// Launch accounting: every kernel launch of the library goes through a Scope, which counts it
// and, when profiling is switched on, brackets it with CUDA events on the launching stream.
#pragma once
#include <cuda_runtime.h>

namespace b2s {
namespace prof {

enum Kind : int {
  K_HIST = 0,     // digit histograms
  K_SCAN,         // histogram scan + pass routing
  K_SWEEP,        // onesweep pass
  K_FIXUP,        // leftovers (copies, synthesised indices)
  K_SEGSORT,      // on-chip segmented sort
  K_UNIT,         // segments of one element
  K_DIST,         // sample / splitter / cut kernels of the distributed sort
  K_MERGE,        // k-way merge
  K_XCHG,         // the partition kernel that writes into the destinations' buffers (or the collective exchange)
  K_COUNT
};

// begin returns the record to hand to end (-1 when timing is off)
int begin(int kind, cudaStream_t stream);
void end(int id, cudaStream_t stream);

// While one of these lives, every launch of the calling thread is accounted under `kind` whatever
// its Scope says (the sort of the gathered samples belongs to the distributed sort's bookkeeping,
// not to the radix passes over the data).
struct Account {
  int saved;
  explicit Account(int kind);
  ~Account();
};

struct Scope {
  int id;
  cudaStream_t stream;
  Scope(int kind, cudaStream_t s) : id(begin(kind, s)), stream(s) {}
  ~Scope() { end(id, stream); }
};

}  // namespace prof
}  // namespace b2s
