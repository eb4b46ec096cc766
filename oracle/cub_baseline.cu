// TEST / MEASUREMENT INFRASTRUCTURE — not part of the product and never linked into
// libb200sort.so.  Only the benchmark and the test-suite may build, load or run this file.
//
// The reference's GPU variant of the SORT task does not have sort kernels of its own: it calls
// the library kernels of NVIDIA CCCL (src/cupynumeric/sort/cub_sort.cuh:57-72 and 118-144:
// cub::DeviceRadixSort::SortKeys / SortPairs; :73-107 and 145-184:
// cub::DeviceSegmentedRadixSort::SortKeys / SortPairs with equal-length segments), after filling
// the index buffer with positions (src/cupynumeric/sort/sort.cu:1851-1862).  This file makes the
// same library calls from the CCCL that ships with the CUDA toolkit of this machine, so that the
// benchmark can time "what the hand-written kernels replace" on the same GPU in the same run.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_segmented_radix_sort.cuh>
#include <cuda_runtime.h>
#include <thrust/iterator/counting_iterator.h>
#include <thrust/iterator/transform_iterator.h>

#include <cstddef>
#include <cstdint>

namespace {

struct TimesSegment {
  long long seg;
  __host__ __device__ long long operator()(long long x) const { return x * seg; }
};

// positions along the sort axis: i (one segment) or i % segment (sort.h:83-92)
__global__ void positions_kernel(int64_t* idx, size_t volume, size_t segment)
{
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < volume; i += stride)
    idx[i] = (int64_t)(segment == volume ? i : i % segment);
}

template <typename T>
cudaError_t run(const void* keys_in, void* keys_out, const int64_t* idx_in, int64_t* idx_out, size_t volume,
                size_t segment, void* temp, size_t* temp_bytes, cudaStream_t stream)
{
  const T* in = static_cast<const T*>(keys_in);
  T* out      = static_cast<T*>(keys_out);
  if (segment == volume) {
    if (idx_out == nullptr)
      return cub::DeviceRadixSort::SortKeys(temp, *temp_bytes, in, out, (long long)volume, 0, (int)sizeof(T) * 8, stream);
    return cub::DeviceRadixSort::SortPairs(temp, *temp_bytes, in, out, idx_in, idx_out, (long long)volume, 0,
                                           (int)sizeof(T) * 8, stream);
  }
  auto begin = thrust::make_transform_iterator(thrust::make_counting_iterator<long long>(0), TimesSegment{(long long)segment});
  auto end   = thrust::make_transform_iterator(thrust::make_counting_iterator<long long>(1), TimesSegment{(long long)segment});
  const long long nseg = (long long)(volume / segment);
  if (idx_out == nullptr)
    return cub::DeviceSegmentedRadixSort::SortKeys(temp, *temp_bytes, in, out, (long long)volume, nseg, begin, end, 0,
                                                   (int)sizeof(T) * 8, stream);
  return cub::DeviceSegmentedRadixSort::SortPairs(temp, *temp_bytes, in, out, idx_in, idx_out, (long long)volume, nseg,
                                                  begin, end, 0, (int)sizeof(T) * 8, stream);
}

cudaError_t dispatch(int dtype, const void* keys_in, void* keys_out, const int64_t* idx_in, int64_t* idx_out,
                     size_t volume, size_t segment, void* temp, size_t* temp_bytes, cudaStream_t stream)
{
  // numbering of b2s_dtype_t (include/b200sort.h)
  switch (dtype) {
    case 4: return run<int32_t>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    case 5: return run<int64_t>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    case 8: return run<uint32_t>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    case 9: return run<uint64_t>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    case 11: return run<float>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    case 12: return run<double>(keys_in, keys_out, idx_in, idx_out, volume, segment, temp, temp_bytes, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace

extern "C" {

// Bytes of temporary storage the library call wants (the "null pointer" query of cub_sort.cuh).
int cubb_temp_bytes(int dtype, size_t volume, size_t segment, int argsort, size_t* bytes)
{
  size_t need = 0;
  int64_t* fake = argsort ? reinterpret_cast<int64_t*>(16) : nullptr;
  const cudaError_t e = dispatch(dtype, nullptr, nullptr, fake, fake, volume, segment, nullptr, &need, nullptr);
  if (e != cudaSuccess) return (int)e;
  *bytes = need;
  return 0;
}

// One SORT task body as the reference's GPU variant runs it: for argsort the position fill, then
// the library sort.  idx_in is scratch for the positions (volume int64), idx_out the result.
int cubb_sort(int dtype, const void* keys_in, void* keys_out, int64_t* idx_in, int64_t* idx_out, size_t volume,
              size_t segment, void* temp, size_t temp_bytes, void* cuda_stream)
{
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (idx_out != nullptr) {
    positions_kernel<<<148 * 8, 256, 0, stream>>>(idx_in, volume, segment);
  }
  const cudaError_t e = dispatch(dtype, keys_in, keys_out, idx_in, idx_out, volume, segment, temp, &temp_bytes, stream);
  return (int)e;
}
}
