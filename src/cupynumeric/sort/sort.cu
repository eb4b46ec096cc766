// GPU variant of the SORT task over libb200sort: the file that takes the place of the reference's
// src/cupynumeric/sort/sort.cu.  Task ID, scalars, stores, dispatch (sort_template.inl:44-120) and
// the meaning of every argument of SortImplBody stay as they are; what the body does with them
// changes: one call into the C ABI of include/b200sort.h per case instead of the CUB / Thrust /
// NCCL code of the reference (sort.cu:63-1784).
//
//   every segment local        -> b2s_local_sort                       (was local_sort, sort.cu:1881-1891)
//   unbound 1-D output         -> b2s_dist_sort_1d, result bound       (was sample_sort_nccl_nd + bind_data, :1896-1930)
//   N-D, sort axis split       -> b2s_dist_sort_nd into the bound output (was sample_sort_nccl_nd + rebalance_data)
//
// Built inside the reference's tree it includes the reference's own headers; with
// -DB2S_SYNTAX_CHECK it compiles against src/third_party_stubs/legate_min.h instead (a syntax
// check only: Legate is an external dependency that this repository does not carry).
#ifdef B2S_SYNTAX_CHECK
#include "legate_min.h"
#else
#include "cupynumeric/sort/sort.h"
#include "cupynumeric/sort/sort_template.inl"
#include "cupynumeric/cuda_help.h"
#endif

#include <unordered_map>

#include "b200sort.h"

namespace cupynumeric {

using namespace legate;

namespace {

int b2s_code(Type::Code c)  // Legate type code -> b2s_dtype_t
{
  switch (c) {
    case Type::Code::BOOL: return B2S_BOOL;
    case Type::Code::INT8: return B2S_INT8;
    case Type::Code::INT16: return B2S_INT16;
    case Type::Code::INT32: return B2S_INT32;
    case Type::Code::INT64: return B2S_INT64;
    case Type::Code::UINT8: return B2S_UINT8;
    case Type::Code::UINT16: return B2S_UINT16;
    case Type::Code::UINT32: return B2S_UINT32;
    case Type::Code::UINT64: return B2S_UINT64;
    case Type::Code::FLOAT16: return B2S_FLOAT16;
    case Type::Code::FLOAT32: return B2S_FLOAT32;
    case Type::Code::FLOAT64: return B2S_FLOAT64;
    case Type::Code::COMPLEX64: return B2S_COMPLEX64;
    case Type::Code::COMPLEX128: return B2S_COMPLEX128;
    default: return 0;
  }
}

// The reference aborts the process on CUDA / NCCL errors (cuda_help.h:238-300); the library
// returns a status instead, so the same behaviour is one line here.
void b2s_check(int status)
{
  if (status != B2S_OK) {
    LEGATE_ABORT(b2s_status_string(status));
  }
}

// Allocator callbacks over the task's framebuffer pool (with_has_allocations, sort.h:98-103): the
// library never allocates device memory itself.
struct PoolCtx {
  std::unordered_map<void*, Buffer<int8_t>> live;
};
void* pool_alloc(void* ctx, size_t bytes)
{
  auto buffer = create_buffer<int8_t>(bytes > 0 ? bytes : 1, Memory::Kind::GPU_FB_MEM, 256);
  void* p     = buffer.ptr(0);
  static_cast<PoolCtx*>(ctx)->live.emplace(p, buffer);
  return p;
}
void pool_free(void* ctx, void* p)
{
  auto& live = static_cast<PoolCtx*>(ctx)->live;
  auto it    = live.find(p);
  if (it != live.end()) {
    it->second.destroy();
    live.erase(it);
  }
}
// the reference brackets every NCCL call with this barrier (sort.cu:1313-1315,1393,1412,...)
void task_barrier(void* ctx) { static_cast<TaskContext*>(ctx)->concurrent_task_barrier(); }

}  // namespace

template <Type::Code CODE, int32_t DIM>
struct SortImplBody<VariantKind::GPU, CODE, DIM> {
  using VAL = type_of<CODE>;

  void operator()(TaskContext& context,
                  const legate::PhysicalStore& input_array,
                  legate::PhysicalStore& output_array,
                  const Pitches<DIM - 1>& /*pitches*/,
                  const Rect<DIM>& rect,
                  const size_t volume,
                  const size_t segment_size_l,
                  const size_t segment_size_g,
                  const bool argsort,
                  const bool stable,
                  const bool is_index_space,
                  const size_t local_rank,
                  const size_t num_ranks,
                  const size_t num_sort_ranks,
                  const std::vector<comm::Communicator>& comms)
  {
    auto stream      = context.get_task_stream();
    const int dtype  = b2s_code(CODE);
    const VAL* in    = volume > 0 ? input_array.read_accessor<VAL, DIM>(rect).ptr(rect.lo) : nullptr;
    const bool unbound               = output_array.is_unbound_store();
    const bool need_distributed_sort = segment_size_l != segment_size_g || unbound;  // sort.cu:1825

    if (!need_distributed_sort) {
      // ---- every segment is local: one call; indices are synthesised inside the first radix pass
      // (lo + i for 1-D, i % L + lo_last for N-D, sort.cu:1851-1862), the input is never copied ----
      if (volume == 0) {
        return;
      }
      size_t ws_bytes = 0;
      b2s_check(b2s_workspace_bytes(dtype, volume, segment_size_l, argsort, &ws_bytes));
      auto ws        = create_buffer<int8_t>(ws_bytes, Memory::Kind::GPU_FB_MEM, 256);
      void* keys_out = argsort ? nullptr : static_cast<void*>(output_array.write_accessor<VAL, DIM>(rect).ptr(rect.lo));
      int64_t* idx   = argsort ? output_array.write_accessor<int64_t, DIM>(rect).ptr(rect.lo) : nullptr;
      b2s_check(b2s_local_sort(dtype, in, keys_out, idx, volume, segment_size_l, rect.lo[DIM - 1], DIM == 1 ? 1 : 0,
                               stable ? 1 : 0, ws.ptr(0), ws_bytes, stream));
      // also reports a bounded device-side wait that ran out (CUPYNUMERIC_CHECK_CUDA_STREAM's place)
      b2s_check(b2s_check_status(ws.ptr(0), stream));
      ws.destroy();
      return;
    }

    PoolCtx pool;
    ncclComm_t comm = is_index_space ? *comms[0].get<ncclComm_t*>() : nullptr;
    const int rank = is_index_space ? static_cast<int>(local_rank) : 0;
    const int size = is_index_space ? static_cast<int>(num_ranks) : 1;

    if (unbound) {
      // ---- 1-D array spanning the GPUs: this rank's part of the global stable sort, bound as the
      // unbound output (sort.cu:1774-1783); a single-GPU launch takes the same call with size 1 ----
      void* out      = nullptr;
      size_t out_len = 0;
      b2s_check(b2s_dist_sort_1d(dtype, in, volume, rect.lo[0], argsort ? 1 : 0, comm, rank, size, pool_alloc, pool_free,
                                 &pool, task_barrier, &context, &out, &out_len, nullptr, stream));
      auto holder = pool.live.at(out);  // ownership of the result passes to Legate
      pool.live.erase(out);
      if (argsort) {
        auto typed = *reinterpret_cast<Buffer<int64_t>*>(&holder);  // same allocation, viewed as the output's type
        output_array.bind_data(typed, Point<1>(static_cast<int64_t>(out_len)));
      } else {
        auto typed = *reinterpret_cast<Buffer<VAL>*>(&holder);
        output_array.bind_data(typed, Point<1>(static_cast<int64_t>(out_len)));
      }
      return;
    }

    // ---- N-D tile whose sort axis is split over the ranks of the launch: all rows in one call, each
    // rank's own extent of every sorted row straight into the bound output ----
    if (num_sort_ranks != num_ranks) {
      // a launch grid with several rows of ranks needs one communicator per row of ranks
      // (ncclCommSplit, kept across calls); not part of this file yet
      LEGATE_ABORT("SORT: sort axis split over a sub-group of the launch is not supported by this build");
    }
    void* out_ptr = nullptr;
    if (volume > 0) {
      out_ptr = argsort ? static_cast<void*>(output_array.write_accessor<int64_t, DIM>(rect).ptr(rect.lo))
                        : static_cast<void*>(output_array.write_accessor<VAL, DIM>(rect).ptr(rect.lo));
    }
    const size_t rows = segment_size_l > 0 ? volume / segment_size_l : 0;
    b2s_check(b2s_dist_sort_nd(dtype, in, out_ptr, argsort ? 1 : 0, rows, segment_size_l, comm, rank, size, pool_alloc,
                               pool_free, &pool, task_barrier, &context, stream));
  }
};

/*static*/ void SortTask::gpu_variant(TaskContext context) { sort_template<VariantKind::GPU>(context); }

}  // namespace cupynumeric

#ifdef B2S_SYNTAX_CHECK
// one instantiation per output kind, so that the syntax check sees the template's body
template struct cupynumeric::SortImplBody<legate::VariantKind::GPU, legate::Type::Code::FLOAT32, 1>;
template struct cupynumeric::SortImplBody<legate::VariantKind::GPU, legate::Type::Code::INT64, 3>;
#endif
