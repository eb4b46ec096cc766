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
  K_XCHG,         // the grouped NCCL send/recv exchange (not a kernel of this library)
  K_COUNT
};

void begin(int kind, cudaStream_t stream);
void end(int kind, cudaStream_t stream);

struct Scope {
  int kind;
  cudaStream_t stream;
  Scope(int k, cudaStream_t s) : kind(k), stream(s) { begin(kind, stream); }
  ~Scope() { end(kind, stream); }
};

}  // namespace prof
}  // namespace b2s
