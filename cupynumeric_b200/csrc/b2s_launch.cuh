// Host-side launchers of the local sort kernels, templated on the key width so that each width
// compiles in a translation unit of its own.
#pragma once

#include "b2s_prof.h"
#include "b2s_radix.cuh"
#include "b2s_segsort.cuh"
#include "b2s_segmerge.cuh"

#include <cstdlib>

namespace b2s {

// Largest segment the on-chip segmented kernel takes.
constexpr unsigned int SEG_CAP = 8192;

// Tile shape of the onesweep pass per key width / payload.
// Tile shapes found by sweeps on B200 (2^28 keys): more keys per thread amortise the per-tile
// work (counter zeroing, row scan, look-back); pairs run three CTAs per SM.
// -DB2S_CFG_<group>_{THREADS,ITEMS,MINCTAS} override a group for tuning sweeps; groups are
// K4 (keys only, <= 4-byte keys), K8 (keys only, 8-byte keys), P4 / P8 (key + index).
#ifndef B2S_CFG_CHAINS
#define B2S_CFG_CHAINS 1
#endif
#ifndef B2S_CFG_K4_THREADS
#define B2S_CFG_K4_THREADS 256
#endif
#ifndef B2S_CFG_K4_ITEMS
#define B2S_CFG_K4_ITEMS 20
#endif
#ifndef B2S_CFG_K4_MINCTAS
#define B2S_CFG_K4_MINCTAS 4
#endif
#ifndef B2S_CFG_K8_THREADS
#define B2S_CFG_K8_THREADS 256
#endif
#ifndef B2S_CFG_K8_ITEMS
#define B2S_CFG_K8_ITEMS 28
#endif
#ifndef B2S_CFG_K8_MINCTAS
#define B2S_CFG_K8_MINCTAS 3
#endif
#ifndef B2S_CFG_P4_THREADS
#define B2S_CFG_P4_THREADS 256
#endif
#ifndef B2S_CFG_P4_ITEMS
#define B2S_CFG_P4_ITEMS 32
#endif
#ifndef B2S_CFG_P4_MINCTAS
#define B2S_CFG_P4_MINCTAS 3
#endif
#ifndef B2S_CFG_P8_THREADS
#define B2S_CFG_P8_THREADS 256
#endif
#ifndef B2S_CFG_P8_ITEMS
#define B2S_CFG_P8_ITEMS 20
#endif
#ifndef B2S_CFG_P8_MINCTAS
#define B2S_CFG_P8_MINCTAS 3
#endif
template <int KB, bool PAIRS> struct SweepCfg {
  static constexpr int THREADS = PAIRS ? (KB == 8 ? B2S_CFG_P8_THREADS : B2S_CFG_P4_THREADS)
                                       : (KB == 8 ? B2S_CFG_K8_THREADS : B2S_CFG_K4_THREADS);
  static constexpr int ITEMS   = PAIRS ? (KB == 8 ? B2S_CFG_P8_ITEMS : B2S_CFG_P4_ITEMS)
                                       : (KB == 8 ? B2S_CFG_K8_ITEMS : B2S_CFG_K4_ITEMS);
  static constexpr int MINCTAS = PAIRS ? (KB == 8 ? B2S_CFG_P8_MINCTAS : B2S_CFG_P4_MINCTAS)
                                       : (KB == 8 ? B2S_CFG_K8_MINCTAS : B2S_CFG_K4_MINCTAS);
  static constexpr int CHAINS  = B2S_CFG_CHAINS;
  static constexpr int TILE    = THREADS * ITEMS;
};

struct Radix1dLayout {
  size_t off_lookback, off_keys[2], off_idx[2], total;
  unsigned int tiles;
};

template <int KB>
inline Radix1dLayout radix_1d_layout(size_t n, bool pairs)
{
  Radix1dLayout l{};
  const unsigned int tile = pairs ? SweepCfg<KB, true>::TILE : SweepCfg<KB, false>::TILE;
  l.tiles                 = (unsigned int)((n + tile - 1) / tile);
  size_t off              = align_up(sizeof(Ctrl), 256);
  l.off_lookback          = off;
  off += align_up((size_t)KB * l.tiles * RADIX * sizeof(unsigned int), 256);
  for (int i = 0; i < 2; ++i) {
    l.off_keys[i] = off;
    off += align_up(n * KB, 256);
  }
  for (int i = 0; i < 2; ++i) {
    l.off_idx[i] = off;
    if (pairs) off += align_up(n * 4, 256);
  }
  l.total = off;
  return l;
}

template <int KB, int XF, bool PAIRS>
inline cudaError_t launch_sweeps(Ctrl* ctrl, unsigned int* lookback, unsigned int tiles, SegGeom geo,
                                 int64_t index_offset, cudaStream_t stream)
{
  using C   = SweepCfg<KB, PAIRS>;
  using S   = SweepSmem<KB, PAIRS, C::THREADS, C::ITEMS, C::CHAINS>;
  auto kern = onesweep_kernel<KB, XF, PAIRS, C::THREADS, C::ITEMS, C::CHAINS, C::MINCTAS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::BYTES);
  if (e != cudaSuccess) return e;
  for (int pass = 0; pass < KB; ++pass) {
    prof::Scope ps(prof::K_SWEEP, stream);
    kern<<<tiles, C::THREADS, S::BYTES, stream>>>(ctrl, lookback + (size_t)pass * tiles * RADIX, pass, geo,
                                                  index_offset);
  }
  return cudaGetLastError();
}

#ifndef B2S_HIST_LANES
#define B2S_HIST_LANES 1
#endif

template <int KB, int XF>
inline cudaError_t radix_1d_xf(const void* in, void* out, int64_t* idx_out, unsigned int n,
                               int64_t index_offset, unsigned char* ws, cudaStream_t stream, int idx32,
                               const uint32_t* idx_in, const unsigned int* hist_parts, int hist_nparts)
{
  using K            = typename KeyOf<KB>::type;
  const bool pairs   = idx_out != nullptr;
  const auto lay     = radix_1d_layout<KB>(n, pairs);
  Ctrl* ctrl         = reinterpret_cast<Ctrl*>(ws);
  unsigned int* lb   = reinterpret_cast<unsigned int*>(ws + lay.off_lookback);
  // control block; the look-back tables too unless the histogram kernel clears them
  const bool own_hist = hist_parts == nullptr;
  cudaError_t e       = cudaMemsetAsync(ws, 0, own_hist ? lay.off_lookback : lay.off_keys[0], stream);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned int per_cta = HIST_THREADS * 16;
  unsigned int hgrid         = (n + per_cta - 1) / per_cta;
  if (hgrid > (unsigned int)sms * 4) hgrid = sms * 4;
  RouteArgs ra{};
  ra.keys_in     = in;
  ra.keys_out    = out;
  ra.idx_out     = idx32 ? nullptr : idx_out;
  ra.idx_out32   = idx32 ? reinterpret_cast<uint32_t*>(idx_out) : nullptr;
  ra.idx_in      = idx_in;
  ra.tmp_keys[0] = ws + lay.off_keys[0];
  ra.tmp_keys[1] = ws + lay.off_keys[1];
  ra.tmp_idx[0]  = reinterpret_cast<uint32_t*>(ws + lay.off_idx[0]);
  ra.tmp_idx[1]  = reinterpret_cast<uint32_t*>(ws + lay.off_idx[1]);
  ra.n           = n;
  ra.npass       = KB;
  ra.key_bytes   = KB;
  ra.zero_ptr    = own_hist ? reinterpret_cast<uint4*>(ws + lay.off_lookback) : nullptr;
  ra.zero_vecs   = own_hist ? (lay.off_keys[0] - lay.off_lookback) / 16 : 0;
  if (hist_parts != nullptr) {
    // the histograms were counted elsewhere (by the ranks that sent this GPU its keys)
    prof::Scope ps(prof::K_SCAN, stream);
    hist_from_parts_kernel<<<1, RADIX, 0, stream>>>(ctrl, hist_parts, hist_nparts, ra);
  } else {
    // digit histograms of all passes; the CTA that finishes last scans them and routes the passes
    prof::Scope ps(prof::K_HIST, stream);
#if B2S_HIST_LANES
    // one CTA per SM with a copy of the tables per lane; inputs too small to give every SM a few
    // thousand keys take the single-table kernel
    if (n >= (unsigned int)sms * HISTL_THREADS * 16) {
      auto kern = hist_lanes_kernel<KB, XF>;
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)HistLanes<KB>::BYTES);
      if (e != cudaSuccess) return e;
      kern<<<sms, HISTL_THREADS, HistLanes<KB>::BYTES, stream>>>(static_cast<const K*>(in), n, ctrl, ra);
    } else
#endif
    hist_kernel<KB, XF><<<hgrid, HIST_THREADS, 0, stream>>>(static_cast<const K*>(in), n, ctrl, ra);
  }
  const SegGeom geo{n, lay.tiles, 1u, KB, nullptr};
  e = pairs ? launch_sweeps<KB, XF, true>(ctrl, lb, lay.tiles, geo, index_offset, stream)
            : launch_sweeps<KB, XF, false>(ctrl, lb, lay.tiles, geo, index_offset, stream);
  if (e != cudaSuccess) return e;
  unsigned int fgrid = (n + 256 * 16 - 1) / (256 * 16);
  if (fgrid > (unsigned int)sms * 8) fgrid = sms * 8;
  {
    prof::Scope ps(prof::K_FIXUP, stream);
    fixup_kernel<<<fgrid, 256, 0, stream>>>(ctrl, n, index_offset);
  }
  return cudaGetLastError();
}

// ---- segments too long for the on-chip kernel: onesweep passes whose tiles stay inside segments ----
struct RadixSegLayout {
  size_t off_lookback, off_seghist, off_keys[2], off_idx[2], total;
  unsigned int tiles_per_seg, tiles;
};

template <int KB>
inline RadixSegLayout radix_seg_layout(size_t seg_len, size_t nseg, bool pairs)
{
  RadixSegLayout l{};
  const unsigned int tile = pairs ? SweepCfg<KB, true>::TILE : SweepCfg<KB, false>::TILE;
  l.tiles_per_seg         = (unsigned int)((seg_len + tile - 1) / tile);
  l.tiles                 = (unsigned int)(l.tiles_per_seg * nseg);
  const size_t volume     = seg_len * nseg;
  size_t off              = align_up(sizeof(Ctrl), 256);
  l.off_lookback          = off;
  off += align_up((size_t)KB * l.tiles * RADIX * sizeof(unsigned int), 256);
  l.off_seghist = off;
  off += align_up(nseg * KB * RADIX * sizeof(unsigned int), 256);
  for (int i = 0; i < 2; ++i) {
    l.off_keys[i] = off;
    off += align_up(volume * KB, 256);
  }
  for (int i = 0; i < 2; ++i) {
    l.off_idx[i] = off;
    if (pairs) off += align_up(volume * 4, 256);
  }
  l.total = off;
  return l;
}

template <int KB, int XF>
inline cudaError_t radix_seg_xf(const void* in, void* out, int64_t* idx_out, unsigned int seg_len, unsigned int nseg,
                                int64_t index_offset, unsigned char* ws, cudaStream_t stream)
{
  using K          = typename KeyOf<KB>::type;
  const bool pairs = idx_out != nullptr;
  const auto lay   = radix_seg_layout<KB>(seg_len, nseg, pairs);
  Ctrl* ctrl       = reinterpret_cast<Ctrl*>(ws);
  unsigned int* lb = reinterpret_cast<unsigned int*>(ws + lay.off_lookback);
  unsigned int* sh = reinterpret_cast<unsigned int*>(ws + lay.off_seghist);
  cudaError_t e    = cudaMemsetAsync(ws, 0, lay.off_keys[0], stream);  // control block, look-back table, histograms
  if (e != cudaSuccess) return e;
  const unsigned int chunks = (seg_len + SEG_HIST_CHUNK - 1) / SEG_HIST_CHUNK;
  {
    prof::Scope ps(prof::K_HIST, stream);
    seg_hist_kernel<KB, XF><<<nseg * chunks, 256, 0, stream>>>(static_cast<const K*>(in), seg_len, chunks, sh);
  }
  {
    prof::Scope ps(prof::K_SCAN, stream);
    seg_scan_kernel<<<nseg * KB, RADIX, 0, stream>>>(sh);
  }
  RouteArgs ra{};
  ra.keys_in     = in;
  ra.keys_out    = out;
  ra.idx_out     = idx_out;
  ra.tmp_keys[0] = ws + lay.off_keys[0];
  ra.tmp_keys[1] = ws + lay.off_keys[1];
  ra.tmp_idx[0]  = reinterpret_cast<uint32_t*>(ws + lay.off_idx[0]);
  ra.tmp_idx[1]  = reinterpret_cast<uint32_t*>(ws + lay.off_idx[1]);
  ra.n           = seg_len * nseg;
  ra.npass       = KB;
  ra.key_bytes   = KB;
  {
    // the global histogram stays empty here, so every pass is routed as active
    prof::Scope ps(prof::K_SCAN, stream);
    scan_route_kernel<<<1, RADIX, 0, stream>>>(ctrl, ra);
  }
  // every pass is active here (empty global histogram), so the only leftover is the copy of an
  // in-place single-pass sort out of its temporary
  const SegGeom geo{seg_len, lay.tiles_per_seg, nseg, KB, sh};
  e = pairs ? launch_sweeps<KB, XF, true>(ctrl, lb, lay.tiles, geo, index_offset, stream)
            : launch_sweeps<KB, XF, false>(ctrl, lb, lay.tiles, geo, index_offset, stream);
  if (e != cudaSuccess) return e;
  if (out != nullptr && out == in) {
    prof::Scope ps(prof::K_FIXUP, stream);
    fixup_kernel<<<148 * 4, 256, 0, stream>>>(ctrl, seg_len * nseg, index_offset);
  }
  return cudaGetLastError();
}

// Segments of more than SEG_CAP elements (each below 2^30, fewer than 2^32 elements in all).
template <int KB>
cudaError_t launch_radix_seg(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len,
                             unsigned int nseg, int64_t index_offset, unsigned char* ws, cudaStream_t stream);

// 1-D stable sort of n < 2^30 keys. `ws` must hold radix_1d_layout<KB>(n, idx_out != null).total bytes.
// idx32 != 0: idx_out points to n uint32 values and receives positions 0..n-1 without the offset.
// idx_in != null: the payload of element i is idx_in[i] instead of i (stable argsort of data that
// already carries 32-bit payloads); the output index is index_offset + payload.
// hist_parts != null: hist_nparts ready-made digit histograms ([part][KB][256]) to add up instead
// of reading the keys for them.
template <int KB>
cudaError_t launch_radix_1d(int xf, const void* in, void* out, int64_t* idx_out, unsigned int n,
                            int64_t index_offset, unsigned char* ws, cudaStream_t stream, int idx32 = 0,
                            const uint32_t* idx_in = nullptr, const unsigned int* hist_parts = nullptr,
                            int hist_nparts = 0);

// Segments of seg_len <= SEG_CAP elements, sorted on chip. `ctrl` must be a zeroed control block.
template <int KB>
cudaError_t launch_segsort(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len,
                           unsigned long long nseg, int64_t index_offset, Ctrl* ctrl, cudaStream_t stream);

template <int KB, bool PAIRS, int THREADS, int ITEMS>
inline cudaError_t segsort_cfg(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len,
                               unsigned long long nseg, int64_t index_offset, Ctrl* ctrl, cudaStream_t stream)
{
  using K   = typename KeyOf<KB>::type;
  using S   = SegSmem<KB, PAIRS, THREADS, ITEMS>;
  auto kern = segsort_kernel<KB, PAIRS, THREADS, ITEMS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::BYTES);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_sm = 1;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, S::BYTES);
  if (per_sm < 1) per_sm = 1;
  unsigned long long grid = (unsigned long long)sms * per_sm;
  if (grid > nseg) grid = nseg;
  {
    prof::Scope ps(prof::K_SEGSORT, stream);
    kern<<<(unsigned int)grid, THREADS, S::BYTES, stream>>>(static_cast<const K*>(in), static_cast<K*>(out),
                                                             idx_out, seg_len, nseg, xf, index_offset, ctrl);
  }
  return cudaGetLastError();
}

// The merge-sort form of the on-chip row sort (4- and 8-byte keys, rows of more than 256 elements).
template <int KB, bool PAIRS, int THREADS>
inline cudaError_t segmerge_cfg(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len,
                                unsigned long long nseg, int64_t index_offset, cudaStream_t stream)
{
  using K   = typename KeyOf<KB>::type;
  using S   = SegMergeSmem<KB, PAIRS, THREADS>;
  auto kern = segmerge_kernel<KB, PAIRS, THREADS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::BYTES);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_sm = 1;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, S::BYTES);
  if (per_sm < 1) per_sm = 1;
  unsigned long long grid = (unsigned long long)sms * per_sm;
  if (grid > nseg) grid = nseg;
  {
    prof::Scope ps(prof::K_SEGSORT, stream);
    kern<<<(unsigned int)grid, THREADS, S::BYTES, stream>>>(static_cast<const K*>(in), static_cast<K*>(out), idx_out, seg_len,
                                                             nseg, xf, index_offset);
  }
  return cudaGetLastError();
}

inline bool seg_merge_enabled()
{
  const char* e = std::getenv("B2S_SEG_MERGE");  // 0: keep every row on the radix kernel (comparisons)
  return e == nullptr || e[0] != '0';
}

template <int KB, bool PAIRS>
inline cudaError_t segsort_pairs(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len,
                                 unsigned long long nseg, int64_t index_offset, Ctrl* ctrl, cudaStream_t stream)
{
  if constexpr (KB == 4 || KB == 8) {
    // keys of a sort are mapped back from their images, which the complex64 image does not allow
    if (seg_len > 256 && (PAIRS || xf != XF_CFLOAT) && seg_merge_enabled()) {
      constexpr int V = SM_VT;
      if (seg_len <= 32 * V) return segmerge_cfg<KB, PAIRS, 32>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
      if (seg_len <= 64 * V) return segmerge_cfg<KB, PAIRS, 64>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
      if (seg_len <= 128 * V) return segmerge_cfg<KB, PAIRS, 128>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
      if (seg_len <= 256 * V) return segmerge_cfg<KB, PAIRS, 256>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
      if (seg_len <= 512 * V) return segmerge_cfg<KB, PAIRS, 512>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
      if constexpr (V == 8) return segmerge_cfg<KB, PAIRS, 1024>(xf, in, out, idx_out, seg_len, nseg, index_offset, stream);
    }
  }
  if (seg_len <= 128) return segsort_cfg<KB, PAIRS, 32, 4>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);
  if (seg_len <= 1024) return segsort_cfg<KB, PAIRS, 128, 8>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);
  if (seg_len <= 4096) return segsort_cfg<KB, PAIRS, 256, 16>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);
  return segsort_cfg<KB, PAIRS, 512, 16>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);
}

#define B2S_INSTANTIATE_KEY_WIDTH(KB, HAS_FLOAT, HAS_CFLOAT)                                                          \
  template <>                                                                                             \
  cudaError_t launch_radix_1d<KB>(int xf, const void* in, void* out, int64_t* idx_out, unsigned int n,    \
                                  int64_t index_offset, unsigned char* ws, cudaStream_t stream, int idx32, \
                                  const uint32_t* idx_in, const unsigned int* hp, int hn)                 \
  {                                                                                                       \
    if (xf == XF_UNSIGNED) return radix_1d_xf<KB, XF_UNSIGNED>(in, out, idx_out, n, index_offset, ws, stream, idx32, idx_in, hp, hn); \
    if (xf == XF_SIGNED) return radix_1d_xf<KB, XF_SIGNED>(in, out, idx_out, n, index_offset, ws, stream, idx32, idx_in, hp, hn); \
    if (HAS_FLOAT && xf == XF_FLOAT)                                                                      \
      return radix_1d_xf<KB, (HAS_FLOAT ? XF_FLOAT : XF_UNSIGNED)>(in, out, idx_out, n, index_offset, ws, stream, idx32, idx_in, hp, hn); \
    if (HAS_CFLOAT && xf == XF_CFLOAT)                                                                    \
      return radix_1d_xf<KB, (HAS_CFLOAT ? XF_CFLOAT : XF_UNSIGNED)>(in, out, idx_out, n, index_offset, ws, stream, idx32, idx_in, hp, hn); \
    return cudaErrorInvalidValue;                                                                         \
  }                                                                                                       \
  template <>                                                                                             \
  cudaError_t launch_radix_seg<KB>(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len, \
                                   unsigned int nseg, int64_t index_offset, unsigned char* ws,           \
                                   cudaStream_t stream)                                                   \
  {                                                                                                       \
    if (xf == XF_UNSIGNED) return radix_seg_xf<KB, XF_UNSIGNED>(in, out, idx_out, seg_len, nseg, index_offset, ws, stream); \
    if (xf == XF_SIGNED) return radix_seg_xf<KB, XF_SIGNED>(in, out, idx_out, seg_len, nseg, index_offset, ws, stream); \
    if (HAS_FLOAT && xf == XF_FLOAT)                                                                      \
      return radix_seg_xf<KB, (HAS_FLOAT ? XF_FLOAT : XF_UNSIGNED)>(in, out, idx_out, seg_len, nseg, index_offset, ws, stream); \
    if (HAS_CFLOAT && xf == XF_CFLOAT)                                                                    \
      return radix_seg_xf<KB, (HAS_CFLOAT ? XF_CFLOAT : XF_UNSIGNED)>(in, out, idx_out, seg_len, nseg, index_offset, ws, stream); \
    return cudaErrorInvalidValue;                                                                         \
  }                                                                                                       \
  template <>                                                                                             \
  cudaError_t launch_segsort<KB>(int xf, const void* in, void* out, int64_t* idx_out, unsigned int seg_len, \
                                 unsigned long long nseg, int64_t index_offset, Ctrl* ctrl,               \
                                 cudaStream_t stream)                                                     \
  {                                                                                                       \
    if ((!HAS_FLOAT && xf == XF_FLOAT) || (!HAS_CFLOAT && xf == XF_CFLOAT)) return cudaErrorInvalidValue; \
    if (idx_out != nullptr)                                                                               \
      return segsort_pairs<KB, true>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);    \
    return segsort_pairs<KB, false>(xf, in, out, idx_out, seg_len, nseg, index_offset, ctrl, stream);     \
  }

}  // namespace b2s
