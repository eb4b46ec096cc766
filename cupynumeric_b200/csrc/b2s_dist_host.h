// Host-side logic of the distributed 1-D sort, shared with the device code: where the samples
// are taken, how the splitters are chosen from them and which destination an element gets.
//
// The scheme is a sample sort like the reference's (src/cupynumeric/sort/sort.cu:1270-1784):
// samples carry (value, rank, position) and order by that triple (sort.h:37-81), so a run of
// equal keys can be cut in the middle and the per-rank results, concatenated in rank order, equal
// one global stable sort.  Differences: the samples are taken from the UNSORTED tile and every
// element is sent to its destination before anything is sorted (the reference sorts, exchanges
// and merges); many more samples per rank, each weighted by the number of elements it stands
// for, so that ragged tiles do not skew the splitters; 64-bit positions and counts everywhere.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __CUDACC__
#define B2S_HD __host__ __device__ __forceinline__
#else
#define B2S_HD inline
#endif

namespace b2s {

// A key in its order-preserving unsigned form; `lo` is used by 16-byte keys only (complex128:
// hi = real part, lo = imaginary part).
struct OKey {
  unsigned long long hi, lo;
};
B2S_HD bool okey_less(const OKey& a, const OKey& b) { return a.hi != b.hi ? a.hi < b.hi : a.lo < b.lo; }
B2S_HD bool okey_equal(const OKey& a, const OKey& b) { return a.hi == b.hi && a.lo == b.lo; }

struct Sample {
  OKey okey;
  long long pos;     // position in the owner's tile (input order)
  long long weight;  // elements of the owner's tile this sample stands for; 0: slot not populated
  int rank;          // owner
  int pad_;
};

// With s samples per bucket the ranks' shares vary by about 1/sqrt(s) (2 % here at 8 ranks).  8192
// samples per rank were measured on 8 GPUs and changed nothing (10.03 vs 10.02 ms per step).
#ifndef B2S_SAMPLES_PER_RANK
#define B2S_SAMPLES_PER_RANK 2048
#endif
constexpr int SAMPLES_PER_RANK = B2S_SAMPLES_PER_RANK;
constexpr int MAX_BUCKETS      = 32;  // one bucket per destination rank

// Sample j (0 <= j < s) of a tile of n >= s elements stands for the elements
// [j*n/s, (j+1)*n/s) and sits in the middle of them.
B2S_HD long long sample_range_start(long long j, long long s, long long n) { return j * n / s; }
B2S_HD long long sample_position(long long j, long long s, long long n)
{
  const long long lo = sample_range_start(j, s, n), hi = sample_range_start(j + 1, s, n);
  return lo + (hi - lo) / 2;
}
B2S_HD long long sample_weight(long long j, long long s, long long n)
{
  return sample_range_start(j + 1, s, n) - sample_range_start(j, s, n);
}

// Triple order of samples; unpopulated samples (weight 0) sort last.
B2S_HD bool sample_less(const Sample& a, const Sample& b)
{
  if ((a.weight == 0) != (b.weight == 0)) return a.weight != 0;
  if (!okey_equal(a.okey, b.okey)) return okey_less(a.okey, b.okey);
  if (a.rank != b.rank) return a.rank < b.rank;
  return a.pos < b.pos;
}

// Cumulative weight at which splitter k (1 <= k < nb) is taken: the first sample, in triple
// order, whose inclusive cumulative weight reaches this.
B2S_HD long long splitter_target(long long k, long long total_weight, long long nb)
{
  const long long t = k * total_weight / nb;
  return t < 1 ? 1 : t;
}

// A splitter as the classification uses it on one rank: the element (key, my rank, pos) lies right of
// the splitter iff key > okey, or key == okey and pos > tie_pos.  tie_pos folds the rank part of
// the triple comparison: -1 when the splitter's owner is a lower rank (all my equal keys lie
// right of it), "infinity" when it is a higher rank (all lie left), the splitter's own position
// when it is mine.  An invalid splitter (no populated sample) has nothing right of it.
struct LocalSplitter {
  OKey okey;
  long long tie_pos;
  int valid;
  int pad_;
};

B2S_HD LocalSplitter localise(const Sample& sp, int my_rank)
{
  LocalSplitter l;
  l.okey    = sp.okey;
  l.valid   = sp.weight != 0;
  l.pad_    = 0;
  l.tie_pos = sp.rank < my_rank ? -1 : (sp.rank > my_rank ? 0x7FFFFFFFFFFFFFFFll : sp.pos);
  return l;
}

B2S_HD bool right_of(const LocalSplitter& s, const OKey& key, long long pos)
{
  if (!s.valid) return false;
  if (!okey_equal(key, s.okey)) return okey_less(s.okey, key);
  return pos > s.tie_pos;
}

// Destination bucket of an element: the number of splitters it lies right of.  `split` holds
// nsplit localised splitters in triple order (right_of is monotone over them).
B2S_HD int bucket_of(const LocalSplitter* split, int nsplit, const OKey& key, long long pos)
{
  int lo = 0, hi = nsplit;  // invariant: right of split[0..lo), not right of split[hi..)
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (right_of(split[mid], key, pos)) lo = mid + 1; else hi = mid;
  }
  return lo;
}

}  // namespace b2s
