// Shared device/host definitions of the sm_100a SORT kernels: key types, the order-preserving
// key transforms, PTX helpers (mbarrier, bulk async copy, relaxed global accesses) and the
// control block that lives at the head of every workspace.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// float32 digit extraction through one floating-point add (see to_ordered)
#ifndef B2S_FLOAT_FADD
#define B2S_FLOAT_FADD 2
#endif

namespace b2s {

// ---------------------------------------------------------------------------------------------
// Key storage types: keys travel through every pass as their ORIGINAL bits; only the digit
// extractor sees the transformed (order-preserving, unsigned) value.
// ---------------------------------------------------------------------------------------------
template <int KB> struct KeyOf;
template <> struct KeyOf<1> { using type = uint8_t; };
template <> struct KeyOf<2> { using type = uint16_t; };
template <> struct KeyOf<4> { using type = uint32_t; };
template <> struct KeyOf<8> { using type = uint64_t; };

// Ordering rule of a dtype.
enum : int {
  XF_UNSIGNED = 0,  // bool, uintN
  XF_SIGNED   = 1,  // intN: flip the sign bit
  XF_FLOAT    = 2,  // IEEE floats: -inf < .. < -0.0 == +0.0 < .. < +inf < every NaN
  XF_CFLOAT   = 3   // complex64 as one 8-byte key: (real, imaginary) lexicographic, each part as XF_FLOAT
};

// Maps raw key bits to an unsigned integer whose natural order is the sort order.
// Floats: every NaN (either sign, any payload) maps to all-ones so that NaNs come last and keep
// their input order; -0.0 maps to the image of +0.0 so the two stay in input order.  The
// reference's CPU variant compares with raw '<' (src/cupynumeric/sort/sort_cpu.inl:64-81),
// under which -0.0 == +0.0; NumPy's sort, the reference tests' oracle, puts NaN last.
template <int KB, int XF>
__host__ __device__ __forceinline__ typename KeyOf<KB>::type to_ordered(typename KeyOf<KB>::type raw)
{
  using K        = typename KeyOf<KB>::type;
  constexpr K SB = (K)((K)1 << (8 * KB - 1));
  if (XF == XF_UNSIGNED) {
    return raw;
  } else if (XF == XF_SIGNED) {
    return (K)(raw ^ SB);
  } else if (XF == XF_CFLOAT) {
    // the real part is the first float in memory (the low word); it is the major key.  NaN-last
    // per part gives NumPy's complex order: a NaN real part after every number, and among equal
    // real parts a NaN imaginary part last.
    const unsigned long long r64 = (unsigned long long)raw;
    const unsigned int re = to_ordered<4, XF_FLOAT>((unsigned int)r64);
    const unsigned int im = to_ordered<4, XF_FLOAT>((unsigned int)(r64 >> 32));
    return (K)(((unsigned long long)re << 32) | im);
  } else {
    // exponent mask: all exponent bits set = inf/NaN
    constexpr K EXP = (KB == 2) ? (K)0x7C00u : (KB == 4) ? (K)0x7F800000u : (K)0x7FF0000000000000ull;
#if defined(__CUDA_ARCH__) && B2S_FLOAT_FADD
    if (KB == 4) {
      // float32 on the device: adding +0.0 turns -0.0 into +0.0 and leaves every other value
      // (denormals included) as it is; then the usual sign flip, and NaNs to all-ones.
      const float f        = __uint_as_float((unsigned int)raw);
      const unsigned int u = __float_as_uint(f + 0.0f);
      const unsigned int m = (unsigned int)((int)u >> 31) | 0x80000000u;
      return (K)(f != f ? 0xFFFFFFFFu : (u ^ m));
    }
#if B2S_FLOAT_FADD >= 2
    if (KB == 8) {
      const double f             = __longlong_as_double((long long)raw);
      const unsigned long long u = (unsigned long long)__double_as_longlong(f + 0.0);
      const unsigned long long m = (unsigned long long)((long long)u >> 63) | 0x8000000000000000ull;
      return (K)(f != f ? ~0ull : (u ^ m));
    }
#endif
#endif
    // straight-line selects: branches here would diverge inside the per-key loops
    const K mag  = (K)(raw & (K)~SB);
    const K mask = (raw & SB) ? (K)~(K)0 : SB;   // negative: flip everything; positive: set the sign
    K o          = (K)(raw ^ mask);
    o            = mag > EXP ? (K)~(K)0 : o;     // NaN
    o            = mag == 0 ? SB : o;            // +0.0 and -0.0
    return o;
  }
}

template <int KB>
__host__ __device__ __forceinline__ typename KeyOf<KB>::type to_ordered_rt(typename KeyOf<KB>::type raw, int xf)
{
  if (xf == XF_UNSIGNED) return to_ordered<KB, XF_UNSIGNED>(raw);
  if (xf == XF_SIGNED) return to_ordered<KB, XF_SIGNED>(raw);
  if (KB == 8 && xf == XF_CFLOAT) return to_ordered<(KB == 8 ? 8 : 4), (KB == 8 ? (int)XF_CFLOAT : (int)XF_UNSIGNED)>(raw);
  if (KB >= 2) return to_ordered<(KB >= 2 ? KB : 2), XF_FLOAT>(raw);
  return raw;
}

// Raw bit pattern whose ordered image is all-ones: pads partial tiles so that the padding
// ranks after every real key of the tile.
template <int KB>
__host__ __device__ __forceinline__ typename KeyOf<KB>::type pad_raw(int xf)
{
  using K = typename KeyOf<KB>::type;
  return xf == XF_UNSIGNED ? (K)~(K)0 : (K)((K)~(K)0 >> 1);
}

// ---------------------------------------------------------------------------------------------
// Control block at the start of a workspace (zeroed by one memset per sort call).
// ---------------------------------------------------------------------------------------------
constexpr int RADIX_BITS = 8;
constexpr int RADIX      = 1 << RADIX_BITS;
constexpr int MAX_PASSES = 8;

struct PassDesc {
  const void* src_keys;
  void* dst_keys;          // nullptr: this pass does not write keys
  // Between passes an index travels as its 32-bit position inside the segment; only the last
  // pass widens it to int64 and adds the caller's offset.
  const uint32_t* src_idx;  // nullptr: positions are synthesised from the element position
  uint32_t* dst_idx32;      // intermediate pass
  int64_t* dst_idx64;       // last pass: the caller's index output
  int active;              // 0: the digit is constant over the whole array, pass is the identity
  int pad_;
};

struct FixDesc {
  const void* copy_src;  // non-null: copy copy_bytes from here to copy_dst
  void* copy_dst;
  unsigned long long copy_bytes;
  int64_t* synth_idx;    // non-null: write index_offset + i (or + widen_src[i])
  uint32_t* synth_idx32; // non-null: write i
  const uint32_t* widen_src;  // with synth_idx: the caller's 32-bit payload takes the place of i
};

struct Ctrl {
  unsigned int status;                  // 0 or a b2s_status_t, written by kernels
  unsigned int abort;                   // set with status; every later wait gives up at once
  unsigned int tile_counter[MAX_PASSES];
  unsigned int hist_done;               // CTAs of the histogram kernel that have added their counts
  unsigned int spin_limit;              // 0: SPIN_LIMIT; else the poll limit of the look-back wait (self-test)
  unsigned int pad_[4];
  unsigned int hist[MAX_PASSES][RADIX]; // digit counts, then (after the scan kernel) exclusive bases
  PassDesc pass[MAX_PASSES];
  FixDesc fix;
};

constexpr unsigned int DEV_ERR_TIMEOUT = 5;  // == B2S_ERR_TIMEOUT

// Upper bound on polls of any device-side wait; on overrun the kernel records DEV_ERR_TIMEOUT,
// raises `abort`, publishes what its successors wait for and returns.
constexpr unsigned int SPIN_LIMIT = 1u << 22;

// ---------------------------------------------------------------------------------------------
// PTX helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned int ld_relaxed(const unsigned int* p)
{
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed(unsigned int* p, unsigned int v)
{
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders generic-proxy accesses to shared memory before later async-proxy (bulk copy) accesses.
__device__ __forceinline__ void fence_proxy_async()
{
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bulk asynchronous copy global -> shared (TMA engine, untiled form).  dst, src and bytes must
// all be multiples of 16.  Completion is signalled on `bar` as transferred bytes.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
      smem_u32(smem_dst)),
    "l"(__cvta_generic_to_global(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
    : "memory");
}
// One bounded attempt: the hardware may park the thread for up to `MBAR_SUSPEND_NS` before it
// answers, so a waiting thread does not spend issue slots polling.
constexpr uint32_t MBAR_SUSPEND_NS = 20000;
constexpr unsigned int MBAR_TRIES  = 1u << 16;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
  uint32_t ok;
  asm volatile(
    "{\n\t.reg .pred p;\n\t"
    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
    "selp.u32 %0, 1, 0, p;\n\t}"
    : "=r"(ok)
    : "r"(smem_u32(bar)), "r"(parity), "r"(MBAR_SUSPEND_NS)
    : "memory");
  return ok != 0;
}
// Bounded wait on an mbarrier phase. Returns false when the limit ran out.  Call it from ONE
// thread and hand the result to the rest of the CTA through a barrier: hundreds of threads
// polling the same mbarrier keep the shared-memory pipe busy for everybody else on the SM.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity)
{
  for (unsigned int i = 0; i < MBAR_TRIES; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

__device__ __forceinline__ unsigned int lanemask_lt()
{
  unsigned int m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Lanes of the warp that hold the same 8-bit digit as the caller (the caller included).
// Built from one ballot per digit bit.  On B200 `match.any` costs time proportional to the number
// of distinct values in the warp (about 60 SM-cycles for 30 distinct digits, measured), five
// times more than eight ballots, so the ballot form is the default.
#ifndef B2S_RANK_MATCH
#define B2S_RANK_MATCH 0
#endif
#ifndef B2S_BALLOT_FORM
#define B2S_BALLOT_FORM 0
#endif
template <int B>
__device__ __forceinline__ void ballot_step(unsigned int d, unsigned int& differs)
{
#if B2S_BALLOT_FORM == 1
  // test-and-vote form: one logic op with a predicate result, one vote, one select, one logic op
  const bool bit          = (d & (1u << B)) != 0;
  const unsigned int bal  = __ballot_sync(0xFFFFFFFFu, bit);
  const unsigned int mine = bit ? 0xFFFFFFFFu : 0u;
  differs |= bal ^ mine;
#else
  // the caller's bit B replicated over a word: 0 or 0xFFFFFFFF
  const int mine         = (int)(d << (31 - B)) >> 31;
  const unsigned int bal = __ballot_sync(0xFFFFFFFFu, mine < 0);
  differs |= bal ^ (unsigned int)mine;
#endif
}

__device__ __forceinline__ unsigned int warp_peers(unsigned int d)
{
#if B2S_RANK_MATCH
  return __match_any_sync(0xFFFFFFFFu, d);
#else
  // A lane differs from the caller in bit b exactly where (ballot_b ^ mine_b) is set, mine_b being
  // the caller's own bit replicated over the word; the peers are the lanes that differ nowhere.
  // The per-bit step is PTX so that it stays a test, a vote and a select.
  unsigned int differs = 0;
#if B2S_BALLOT_FORM == 1
  asm volatile("" : "+r"(d));  // keep the digit in a register of its own
#endif
  ballot_step<0>(d, differs);
  ballot_step<1>(d, differs);
  ballot_step<2>(d, differs);
  ballot_step<3>(d, differs);
  ballot_step<4>(d, differs);
  ballot_step<5>(d, differs);
  ballot_step<6>(d, differs);
  ballot_step<7>(d, differs);
  return ~differs;
#endif
}

// Digit extraction with the per-pass constants hoisted out of the per-key work.
struct DigitSel {
  unsigned int prmt;   // byte-permute selector that moves the pass's byte to bits 0..7
  unsigned int flip;   // xor applied to the extracted byte (sign bit of signed keys, top pass only)
  int hi_word;         // 64-bit keys: the digit lives in the upper word
};
template <int KB, int XF>
__device__ __forceinline__ DigitSel make_digit_sel(int pass)
{
  DigitSel s;
  s.prmt    = 0x4440u | (unsigned int)(pass & 3);
  s.flip    = (XF == XF_SIGNED && pass == KB - 1) ? 0x80u : 0u;
  s.hi_word = pass >= 4;
  return s;
}
template <int KB, int XF>
__device__ __forceinline__ unsigned int digit_fast(typename KeyOf<KB>::type raw, const DigitSel& s, int shift)
{
  if (XF == XF_FLOAT) {
    return (unsigned int)(to_ordered<KB, XF>(raw) >> shift) & (RADIX - 1);
  } else if (XF == XF_CFLOAT) {
    // passes 0-3 look at the imaginary part (high word in memory), passes 4-7 at the real part
    const unsigned long long r64 = (unsigned long long)raw;
    const unsigned int w         = s.hi_word ? (unsigned int)r64 : (unsigned int)(r64 >> 32);
    return (to_ordered<4, XF_FLOAT>(w) >> (shift & 31)) & (RADIX - 1);
  } else if (KB == 8) {
    const unsigned long long r64 = (unsigned long long)raw;
    const unsigned int w         = s.hi_word ? (unsigned int)(r64 >> 32) : (unsigned int)r64;
    return __byte_perm(w, 0u, s.prmt) ^ s.flip;
  } else if (KB == 4) {
    return __byte_perm((unsigned int)raw, 0u, s.prmt) ^ s.flip;
  } else {
    return (((unsigned int)raw >> shift) & (RADIX - 1)) ^ s.flip;
  }
}

__device__ __forceinline__ void raise_timeout(Ctrl* ctrl)
{
  atomicMax(&ctrl->status, DEV_ERR_TIMEOUT);
  atomicExch(&ctrl->abort, 1u);
}

template <int KB, int XF>
__device__ __forceinline__ unsigned int digit_of(typename KeyOf<KB>::type raw, int shift)
{
  return (unsigned int)(to_ordered<KB, XF>(raw) >> shift) & (RADIX - 1);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace b2s
