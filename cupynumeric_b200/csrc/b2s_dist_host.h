// Host-side logic of the distributed 1-D sort, shared with the device code: regular sampling,
// splitter selection and the rule that cuts a rank's sorted data at a splitter.
//
// Follows the scheme of the reference's sample sort (src/cupynumeric/sort/sort.cu:1270-1784):
// samples carry (value, rank, position) and order by that triple (sort.h:37-81), so a run of
// equal keys can be cut in the middle and the per-rank results, concatenated in rank order,
// equal one global stable sort.  Differences: many more samples per rank (balance within a few
// per cent instead of the reference's "worst case ... imbalance of x2", sort.cu:1349-1350), and
// 64-bit positions and counts everywhere.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __CUDACC__
#define B2S_HD __host__ __device__ __forceinline__
#else
#define B2S_HD inline
#endif

namespace b2s {

struct Sample {
  unsigned long long okey;  // key in its order-preserving unsigned form
  long long pos;            // position in the owner's locally sorted data
  int rank;                 // owner
  int valid;                // 0: slot not populated (owner has fewer elements than samples)
};

constexpr int SAMPLES_PER_RANK = 256;

// Position of regular sample j (0 <= j < s) in n sorted elements, n >= s: the last element of
// the j-th of s equal chunks.
B2S_HD long long sample_position(long long j, long long s, long long n) { return (j + 1) * n / s - 1; }

// Triple order of samples; unpopulated samples sort last.
B2S_HD bool sample_less(const Sample& a, const Sample& b)
{
  if (a.valid != b.valid) return a.valid > b.valid;
  if (a.okey != b.okey) return a.okey < b.okey;
  if (a.rank != b.rank) return a.rank < b.rank;
  return a.pos < b.pos;
}

// Index (into the sorted, populated samples) of splitter k, 1 <= k < nranks.
B2S_HD long long splitter_index(long long k, long long populated, long long nranks)
{
  long long i = k * populated / nranks - 1;
  return i < 0 ? 0 : i;
}

// Number of leading elements of rank `my_rank`'s sorted data that belong left of `splitter`,
// i.e. whose (key, rank, position) triple is <= the splitter's.  `lower` / `upper` are the
// counts of local keys < and <= the splitter's key.
B2S_HD long long cut_position(const Sample& splitter, int my_rank, long long lower, long long upper)
{
  if (my_rank < splitter.rank) return upper;
  if (my_rank > splitter.rank) return lower;
  return splitter.pos + 1;
}

}  // namespace b2s
