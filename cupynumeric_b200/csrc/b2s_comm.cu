// The collectives the distributed sort needs, behind the b2s_comm_ops table of the C ABI, in two
// forms: over an NCCL communicator (one process per GPU, the production form; the reference's
// task receives its ncclComm_t from Legate, src/cupynumeric/sort/sort.cu:1923) and between the
// threads of one process (ranks that share an address space, synchronised on the host).
#include <cuda_runtime.h>
#include <nccl.h>

#include <condition_variable>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/b200sort.h"

namespace {

// ---- NCCL ----------------------------------------------------------------------------------
struct NcclCtx {
  ncclComm_t comm;
  int rank, nranks;
  int* flag;  // one device int for the barrier, owned by this table
};

int nccl_all_gather(void* c, const void* send, void* recv, size_t bytes, void* stream)
{
  NcclCtx* x = static_cast<NcclCtx*>(c);
  return ncclAllGather(send, recv, bytes, ncclUint8, x->comm, static_cast<cudaStream_t>(stream)) == ncclSuccess
           ? B2S_OK
           : B2S_ERR_NCCL;
}

int nccl_barrier(void* c, void* stream)
{
  NcclCtx* x = static_cast<NcclCtx*>(c);
  return ncclAllReduce(x->flag, x->flag, 1, ncclInt32, ncclSum, x->comm, static_cast<cudaStream_t>(stream)) == ncclSuccess
           ? B2S_OK
           : B2S_ERR_NCCL;
}

int nccl_exchange(void* c, const void* const* send_ptr, const size_t* send_bytes, void* const* recv_ptr,
                  const size_t* recv_bytes, void* stream)
{
  NcclCtx* x     = static_cast<NcclCtx*>(c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (ncclGroupStart() != ncclSuccess) return B2S_ERR_NCCL;
  bool ok = true;
  for (int i = 1; i < x->nranks; ++i) {
    const int to = (x->rank + i) % x->nranks, from = (x->rank - i + x->nranks) % x->nranks;
    if (send_bytes[to] > 0) ok = ok && ncclSend(send_ptr[to], send_bytes[to], ncclUint8, to, x->comm, s) == ncclSuccess;
    if (recv_bytes[from] > 0) ok = ok && ncclRecv(recv_ptr[from], recv_bytes[from], ncclUint8, from, x->comm, s) == ncclSuccess;
  }
  // an opened group is always closed, whatever happened inside it
  ok = (ncclGroupEnd() == ncclSuccess) && ok;
  return ok ? B2S_OK : B2S_ERR_NCCL;
}

// ---- threads of one process ------------------------------------------------------------------
struct ThreadShared {
  int nranks;
  std::mutex mu;
  std::condition_variable cv;
  int arrived          = 0;
  unsigned long long generation = 0;
  int refs;
  // what every rank published for the collective in flight
  std::vector<const void*> send;
  std::vector<const void* const*> send_list;
  std::vector<const size_t*> send_sizes;
  explicit ThreadShared(int n) : nranks(n), refs(n), send(n), send_list(n), send_sizes(n) {}
  void wait_all()
  {
    std::unique_lock<std::mutex> lock(mu);
    const unsigned long long gen = generation;
    if (++arrived == nranks) {
      arrived = 0;
      ++generation;
      cv.notify_all();
    } else {
      cv.wait(lock, [&] { return generation != gen; });
    }
  }
};

struct ThreadCtx {
  ThreadShared* shared;
  int rank;
};

// Every collective here has the same shape: finish my own stream (what I publish is final),
// meet the others, copy what they published, finish the copies, meet again (so that nobody
// reuses a published buffer while somebody still reads it).
int thread_all_gather(void* c, const void* send, void* recv, size_t bytes, void* stream)
{
  ThreadCtx* x   = static_cast<ThreadCtx*>(c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc         = cudaStreamSynchronize(s) == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
  x->shared->send[x->rank] = send;
  x->shared->wait_all();
  for (int p = 0; p < x->shared->nranks && rc == B2S_OK; ++p) {
    unsigned char* dst = static_cast<unsigned char*>(recv) + (size_t)p * bytes;
    if (dst != x->shared->send[p] &&
        cudaMemcpyAsync(dst, x->shared->send[p], bytes, cudaMemcpyDefault, s) != cudaSuccess)
      rc = B2S_ERR_CUDA;
  }
  if (cudaStreamSynchronize(s) != cudaSuccess) rc = B2S_ERR_CUDA;
  x->shared->wait_all();
  return rc;
}

int thread_barrier(void* c, void* stream)
{
  ThreadCtx* x = static_cast<ThreadCtx*>(c);
  const int rc = cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
  x->shared->wait_all();
  return rc;
}

int thread_exchange(void* c, const void* const* send_ptr, const size_t* send_bytes, void* const* recv_ptr,
                    const size_t* recv_bytes, void* stream)
{
  ThreadCtx* x   = static_cast<ThreadCtx*>(c);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc         = cudaStreamSynchronize(s) == cudaSuccess ? B2S_OK : B2S_ERR_CUDA;
  x->shared->send_list[x->rank]  = send_ptr;
  x->shared->send_sizes[x->rank] = send_bytes;
  x->shared->wait_all();
  for (int p = 0; p < x->shared->nranks && rc == B2S_OK; ++p) {
    if (p == x->rank || recv_bytes[p] == 0) continue;
    if (x->shared->send_sizes[p][x->rank] != recv_bytes[p]) {
      rc = B2S_ERR_INVALID_ARG;  // the two sides disagree on a transfer's size
      break;
    }
    if (cudaMemcpyAsync(recv_ptr[p], x->shared->send_list[p][x->rank], recv_bytes[p], cudaMemcpyDefault, s) != cudaSuccess)
      rc = B2S_ERR_CUDA;
  }
  if (cudaStreamSynchronize(s) != cudaSuccess) rc = B2S_ERR_CUDA;
  x->shared->wait_all();
  return rc;
}

}  // namespace

extern "C" {

int b2s_nccl_comm_ops(b2s_comm_ops* ops, void* nccl_comm, int rank, int nranks, void* barrier_word)
{
  if (ops == nullptr || nccl_comm == nullptr || barrier_word == nullptr || nranks < 1 || rank < 0 || rank >= nranks)
    return B2S_ERR_INVALID_ARG;
  NcclCtx* x = new NcclCtx{static_cast<ncclComm_t>(nccl_comm), rank, nranks, static_cast<int*>(barrier_word)};
  ops->ctx        = x;
  ops->all_gather = nccl_all_gather;
  ops->barrier    = nccl_barrier;
  ops->exchange   = nccl_exchange;
  return B2S_OK;
}

void b2s_nccl_comm_ops_release(b2s_comm_ops* ops)
{
  if (ops == nullptr || ops->ctx == nullptr) return;
  delete static_cast<NcclCtx*>(ops->ctx);
  ops->ctx = nullptr;
}

int b2s_thread_comm_create(int nranks, b2s_comm_ops* ops_out)
{
  if (nranks < 1 || ops_out == nullptr) return B2S_ERR_INVALID_ARG;
  ThreadShared* sh = new ThreadShared(nranks);
  for (int r = 0; r < nranks; ++r) {
    ops_out[r].ctx          = new ThreadCtx{sh, r};
    ops_out[r].all_gather   = thread_all_gather;
    ops_out[r].barrier      = thread_barrier;
    ops_out[r].exchange     = thread_exchange;
  }
  return B2S_OK;
}

void b2s_thread_comm_destroy(b2s_comm_ops* ops)
{
  if (ops == nullptr || ops->ctx == nullptr) return;
  ThreadCtx* x     = static_cast<ThreadCtx*>(ops->ctx);
  ThreadShared* sh = x->shared;
  bool last;
  {
    std::lock_guard<std::mutex> lock(sh->mu);
    last = --sh->refs == 0;
  }
  delete x;
  ops->ctx = nullptr;
  if (last) delete sh;
}
}
