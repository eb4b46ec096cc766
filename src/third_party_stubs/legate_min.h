// Stand-in declarations for a syntax check of src/cupynumeric/sort/sort.cu without Legate: only
// the names that file uses, with the shapes they have in Legate and in the reference's headers
// (legate.h; src/cupynumeric/sort/sort.h:27-113; src/cupynumeric/pitches.h; cuda_help.h).  Nothing
// here has behaviour; it is never linked.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <vector>

typedef struct CUstream_st* cudaStream_t;
typedef struct ncclComm* ncclComm_t;
#define LEGATE_ABORT(msg) std::abort()

namespace legate {
enum class VariantKind : int { CPU, OMP, GPU };
struct Type {
  enum class Code : int { BOOL, INT8, INT16, INT32, INT64, UINT8, UINT16, UINT32, UINT64, FLOAT16, FLOAT32, FLOAT64, COMPLEX64, COMPLEX128 };
};
template <Type::Code CODE> struct type_of_impl { using type = int64_t; };
template <Type::Code CODE> using type_of = typename type_of_impl<CODE>::type;
template <int DIM> struct Point {
  int64_t v[DIM > 0 ? DIM : 1];
  Point() = default;
  explicit Point(int64_t x) { v[0] = x; }
  int64_t& operator[](int i) { return v[i]; }
  const int64_t& operator[](int i) const { return v[i]; }
};
template <int DIM> struct Rect {
  Point<DIM> lo, hi;
  bool empty() const;
};
struct Memory { enum class Kind : int { GPU_FB_MEM, Z_COPY_MEM }; };
template <typename T, int DIM = 1> struct Buffer {
  T* ptr(const Point<DIM>&) const;
  T* ptr(int64_t) const;
  void destroy();
};
template <typename T> Buffer<T> create_buffer(size_t n, Memory::Kind kind, size_t alignment = 16);
template <typename T, int DIM> struct AccessorRO { const T* ptr(const Point<DIM>&) const; };
template <typename T, int DIM> struct AccessorWO { T* ptr(const Point<DIM>&) const; };
struct PhysicalStore {
  template <typename T, int DIM> AccessorRO<T, DIM> read_accessor(const Rect<DIM>&) const;
  template <typename T, int DIM> AccessorWO<T, DIM> write_accessor(const Rect<DIM>&) const;
  bool is_unbound_store() const;
  template <typename T> void bind_data(Buffer<T>& buffer, const Point<1>& extents);
  void bind_empty_data();
};
namespace comm {
struct Communicator { template <typename T> T get() const; };
}  // namespace comm
struct TaskContext {
  cudaStream_t get_task_stream() const;
  void concurrent_task_barrier();
};
}  // namespace legate

namespace cupynumeric {
using namespace legate;
template <int DIM> struct Pitches { size_t flatten(const Rect<DIM + 1>&); };
template <> struct Pitches<0> { size_t flatten(const Rect<1>&); };
template <VariantKind KIND, Type::Code CODE, int32_t DIM> struct SortImplBody;
struct SortTask { static void gpu_variant(legate::TaskContext context); };
template <VariantKind KIND> static void sort_template(legate::TaskContext& context);  // sort_template.inl:92-120
}  // namespace cupynumeric
