// TEST INFRASTRUCTURE — CPU oracle for the SORT task. Not part of the product:
// only the test-suite, the smoke check and the benchmark's CPU-baseline /
// reference arm may build, load or run this file.
//
// It restates, call for call, the arithmetic of the reference's CPU and OpenMP
// SORT variants, which is a handful of Thrust calls:
//   src/cupynumeric/sort/sort_cpu.inl:52-85   thrust_local_sort_inplace
//       (per segment: thrust::stable_sort / thrust::sort /
//        thrust::stable_sort_by_key / thrust::sort_by_key with ::cuda::std::less{})
//   src/cupynumeric/sort/sort_cpu.inl:990-1002 argsort index initialisation
//       (1-D: lo + i ; N-D: i % L + lo_last, functor sort.h:83-92)
//   src/cupynumeric/sort/sort_cpu.inl:1020-1026 copy input -> working buffer
//   src/cupynumeric/sort/sort.cc:64 (thrust::host) and sort_omp.cc:65 (thrust::omp::par)
// The sorting itself lives in a third-party dependency that the reference does
// not vendor: NVIDIA CCCL/Thrust (host "cpp" and "omp" backends). Its version is
// pinned inside Legate's build (Legate pinned at cmake/versions.json:3-15); the
// copy used here is the CCCL 2.8.2 that ships with CUDA 12.9.
//
// Pinning: the unit tests check this oracle against every golden vector held
// by the reference's own tests for this path (tests/cpp/integration/test_sort.cc,
// test_argsort.cc) and against NumPy's stable sort, which is the reference's
// own test oracle (tests/integration/test_sort.py:85-102).
//
// NaN: the literal reference comparator (raw '<') is not a strict weak order
// when NaNs are present, and the reference has no test with NaN input, so NaN
// placement is PARITY UNPINNED at this boundary. With nan_mode = 1 the
// comparator is replaced by "a < b, NaN greater than every number, NaN
// equivalent to NaN" (NumPy's NaN-last order); with nan_mode = 0 the literal
// reference comparator runs. Both agree bit for bit on NaN-free input.
#include <thrust/execution_policy.h>
#include <thrust/sort.h>
#include <thrust/system/omp/execution_policy.h>
#include <cuda/std/functional>

#include <algorithm>
#include <cmath>
#include <complex>
#include <cstdint>
#include <cstring>

namespace {

enum DType : int {
  DT_BOOL = 1, DT_INT8, DT_INT16, DT_INT32, DT_INT64, DT_UINT8, DT_UINT16, DT_UINT32, DT_UINT64,
  DT_FLOAT16, DT_FLOAT32, DT_FLOAT64, DT_COMPLEX64, DT_COMPLEX128
};

// IEEE binary16 held as bits; ordering goes through float exactly like __half's host operator<.
struct half_t {
  uint16_t bits;
};
inline float half_to_float(half_t h)
{
  uint32_t s = (h.bits >> 15) & 1u, e = (h.bits >> 10) & 0x1Fu, m = h.bits & 0x3FFu, out;
  if (e == 0) {
    if (m == 0) {
      out = s << 31;
    } else {
      int sh = 0;
      while (!(m & 0x400u)) { m <<= 1; ++sh; }
      m &= 0x3FFu;
      out = (s << 31) | ((uint32_t)(127 - 15 - sh + 1) << 23) | (m << 13);
    }
  } else if (e == 31) {
    out = (s << 31) | 0x7F800000u | (m << 13);
  } else {
    out = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
  }
  float f;
  std::memcpy(&f, &out, 4);
  return f;
}
inline bool operator<(half_t a, half_t b) { return half_to_float(a) < half_to_float(b); }

// Complex ordering of the reference: lexicographic on (real, imag)
// (src/cupynumeric/binary/binary_op_util.h:32-36 as used by the sort comparators).
template <typename F>
struct cplx {
  F re, im;
};
template <typename F>
inline bool operator<(cplx<F> a, cplx<F> b)
{
  return a.re < b.re || (a.re == b.re && a.im < b.im);
}

template <typename T> inline bool is_nan(T) { return false; }
inline bool is_nan(float v) { return v != v; }
inline bool is_nan(double v) { return v != v; }
inline bool is_nan(half_t v) { float f = half_to_float(v); return f != f; }

template <typename T>
struct nan_last_less {
  bool operator()(const T& a, const T& b) const
  {
    if (is_nan(a)) return false;
    if (is_nan(b)) return true;
    return a < b;
  }
};

// sort_cpu.inl:52-85, verbatim structure; COMP is ::cuda::std::less<> for the literal reference.
template <typename VAL, typename Policy, typename COMP>
void local_sort_inplace(VAL* inptr, int64_t* argptr, size_t volume, size_t sort_dim_size,
                        bool stable_argsort, const Policy& exec, COMP comp)
{
  if (sort_dim_size == 0) return;
  if (argptr == nullptr) {
    for (size_t start_idx = 0; start_idx < volume; start_idx += sort_dim_size) {
      if (stable_argsort) {
        thrust::stable_sort(exec, inptr + start_idx, inptr + start_idx + sort_dim_size, comp);
      } else {
        thrust::sort(exec, inptr + start_idx, inptr + start_idx + sort_dim_size, comp);
      }
    }
  } else {
    for (uint64_t start_idx = 0; start_idx < volume; start_idx += sort_dim_size) {
      int64_t* segmentValues = argptr + start_idx;
      VAL* segmentKeys       = inptr + start_idx;
      if (stable_argsort) {
        thrust::stable_sort_by_key(exec, segmentKeys, segmentKeys + sort_dim_size, segmentValues, comp);
      } else {
        thrust::sort_by_key(exec, segmentKeys, segmentKeys + sort_dim_size, segmentValues, comp);
      }
    }
  }
}

template <typename VAL>
int run(VAL* keys, int64_t* idx, size_t volume, size_t segment, int64_t index_offset, int ndim_is_1,
        int stable, int backend, int nan_mode)
{
  if (idx != nullptr) {
    // sort_cpu.inl:990-1002
    if (ndim_is_1) {
      for (size_t i = 0; i < volume; ++i) idx[i] = index_offset + (int64_t)i;
    } else {
      for (size_t i = 0; i < volume; ++i) idx[i] = (int64_t)(i % segment) + index_offset;
    }
  }
  if (volume == 0) return 0;
  if (nan_mode == 1) {
    nan_last_less<VAL> comp;
    if (backend == 1) local_sort_inplace(keys, idx, volume, segment, stable != 0, thrust::omp::par, comp);
    else local_sort_inplace(keys, idx, volume, segment, stable != 0, thrust::host, comp);
  } else {
    ::cuda::std::less<> comp{};
    if (backend == 1) local_sort_inplace(keys, idx, volume, segment, stable != 0, thrust::omp::par, comp);
    else local_sort_inplace(keys, idx, volume, segment, stable != 0, thrust::host, comp);
  }
  return 0;
}

}  // namespace

extern "C" {

// keys: working buffer holding a COPY of the input (sorted in place, as the reference does
// after its std::copy). idx: nullptr for sort, else `volume` int64 written here.
// segment: extent of the sort (last) axis. ndim_is_1: selects the index initialisation rule.
// backend: 0 = thrust::host (CPU variant), 1 = thrust::omp::par (OMP variant).
// nan_mode: 0 = literal reference comparator, 1 = NaN-last comparator.
// Returns 0, or -1 for an unknown dtype.
int oracle_sort(int dtype, void* keys, int64_t* idx, size_t volume, size_t segment,
                int64_t index_offset, int ndim_is_1, int stable, int backend, int nan_mode)
{
  switch (dtype) {
    case DT_BOOL: return run((uint8_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_INT8: return run((int8_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_INT16: return run((int16_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_INT32: return run((int32_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_INT64: return run((int64_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_UINT8: return run((uint8_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_UINT16: return run((uint16_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_UINT32: return run((uint32_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_UINT64: return run((uint64_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_FLOAT16: return run((half_t*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_FLOAT32: return run((float*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_FLOAT64: return run((double*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_COMPLEX64: return run((cplx<float>*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    case DT_COMPLEX128: return run((cplx<double>*)keys, idx, volume, segment, index_offset, ndim_is_1, stable, backend, nan_mode);
    default: return -1;
  }
}

int oracle_thrust_version(void) { return THRUST_VERSION; }
}

#include <omp.h>
extern "C" int oracle_num_threads(void) { return omp_get_max_threads(); }
// Threads of the OpenMP back-end from now on (launchers such as torch.distributed.run export
// OMP_NUM_THREADS=1 to their children; the benchmark's reference arm undoes that here).
extern "C" void oracle_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }
