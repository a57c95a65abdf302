// Stable LSD radix sort of (32-bit key, lookup position) pairs, shared by the segment-reduce and the owner routing.
//
// One pass = a per-tile digit histogram kernel and a scatter kernel.  While tiles x digits is small the scatter kernel
// derives its tile's offsets itself (sum of the earlier tiles + scan of the digit totals); larger problems scan the
// histogram with a single-CTA kernel in between.
#pragma once
#include "common.cuh"
#include "scan.cuh"

namespace srm2 {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortRounds = 4;                               // elements per thread
constexpr int kSortTile = kSortThreads * kSortRounds;        // 1024 elements per CTA
constexpr int kMaxRadixBits = 11;
constexpr int kSuperTile = 16;                               // tiles per group whose digit sums are kept as well
constexpr int64_t kFusedOffsetsLimit = (int64_t)1 << 23;     // tiles * digits up to which the scatter kernel derives its offsets itself

// Key of a 64-bit input value: mod == 0: the value itself, with anything outside [0, cap) mapped to `cap` (behind every
// real key); mod > 0: value mod `mod` (owner of a row id), negative values mapped to 0.
__device__ __forceinline__ uint32_t make_key(int64_t k, int64_t cap, int mod) {
  if (mod > 0) return k < 0 ? 0u : (uint32_t)(k % mod);
  return (k < 0 || k >= cap) ? (uint32_t)cap : (uint32_t)k;
}

// Histogram of one digit per tile.  Pass 0 reads the keys from the int64 source array (key32 == nullptr), later passes
// from the u32 ping-pong buffer.  Two layouts:
//   dtot != nullptr: tile-major hist[tile * bins + d] (coalesced); the digit totals are accumulated into dtot[d] and the
//                    sums of every group of kSuperTile tiles into dtot[(1 + group) * bins + d] (integer atomics: the
//                    result does not depend on their order); the scatter kernel adds the groups and the tiles before
//                    its own and scans the totals itself — no scan launch;
//   dtot == nullptr: digit-major hist[d * tiles + tile], to be scanned by a separate kernel (large problems).
static __global__ void __launch_bounds__(kSortThreads)
srm2_sort_hist_kernel(const int64_t* __restrict__ key64, const uint32_t* __restrict__ key32, int64_t n_host,
                      const int64_t* __restrict__ n_dev, int shift, int bits,
                      uint32_t* __restrict__ hist, uint32_t* __restrict__ dtot, int tiles, int64_t cap, int mod) {
  extern __shared__ uint32_t sh[];
  const int64_t n = eff_count(n_host, n_dev);
  const int bins = 1 << bits;
  for (int b = threadIdx.x; b < bins; b += kSortThreads) sh[b] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < n) {
      const uint32_t k = key64 ? make_key(key64[i], cap, mod) : key32[i];
      atomicAdd(&sh[(k >> shift) & (bins - 1)], 1u);
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kSortThreads) {
    const uint32_t c = sh[b];
    if (dtot) {
      hist[(int64_t)blockIdx.x * bins + b] = c;
      if (c) { atomicAdd(dtot + b, c); atomicAdd(dtot + (int64_t)(1 + blockIdx.x / kSuperTile) * bins + b, c); }
    }
    else hist[(int64_t)b * tiles + blockIdx.x] = c;
  }
}

// Stable scatter of one tile.  Warp w owns elements [w*128, (w+1)*128) of the tile and walks them in rounds of 32
// consecutive elements; __match_any_sync groups equal digits of a round, so the rank of an element among the equal
// digits of its warp's sub-range is (count so far) + (equal digits in lower lanes).  Warp counts are then scanned
// across the warps of the tile and added to the tile's global digit offset.
// dtot != nullptr: hist is the raw tile-major histogram and dtot the digit totals (see the histogram kernel);
// dtot == nullptr: hist holds the exclusive scan of the whole digit-major histogram.
static __global__ void __launch_bounds__(kSortThreads)
srm2_sort_scatter_kernel(const int64_t* __restrict__ key64, const uint32_t* __restrict__ key32,
                         const uint32_t* __restrict__ val32, int64_t n_host, const int64_t* __restrict__ n_dev, int shift, int bits,
                         const uint32_t* __restrict__ hist, const uint32_t* __restrict__ dtot, int tiles, uint32_t* __restrict__ out_key,
                         uint32_t* __restrict__ out_val, int64_t cap, int mod) {
  extern __shared__ uint32_t sh[];
  const int64_t n = eff_count(n_host, n_dev);                 // [kSortWarps][bins] counts, [bins] tile offsets
  __shared__ uint32_t ws[33];
  const int bins = 1 << bits;
  uint32_t* goff = sh + kSortWarps * bins;         // global offset of (digit, this tile)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int b = threadIdx.x; b < bins * kSortWarps; b += kSortThreads) sh[b] = 0;
  // ---- this warp's keys and positions, all loads issued before anything depends on them ----
  const int64_t base_i = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (32 * kSortRounds);
  uint32_t key[kSortRounds], val[kSortRounds], rnk[kSortRounds];
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base_i + r * 32 + lane;
    key[r] = 0; val[r] = (uint32_t)i;
    if (i < n) {
      key[r] = key64 ? make_key(key64[i], cap, mod) : key32[i];
      if (val32) val[r] = val32[i];
    }
  }
  // ---- global offsets of this tile's digits ----
  if (dtot == nullptr) {
    for (int b = threadIdx.x; b < bins; b += kSortThreads) goff[b] = hist[(int64_t)b * tiles + blockIdx.x];
  } else {
    // thread t owns the consecutive digits [t*per, (t+1)*per): sum of the earlier tiles (coalesced over threads when
    // per == 1, i.e. up to 256 digits; still line-friendly above), then a block scan of the digit totals
    const int per = (bins + kSortThreads - 1) / kSortThreads;
    uint32_t tsum = 0;
    for (int q = 0; q < per; ++q) {
      const int b = threadIdx.x * per + q;
      if (b >= bins) break;
      const uint32_t* col = hist + b;
      uint32_t before = 0;
      const int my_group = (int)blockIdx.x / kSuperTile;
      for (int gq = 0; gq < my_group; ++gq) before += __ldg(dtot + (int64_t)(1 + gq) * bins + b);
      int t = my_group * kSuperTile;
      for (; t + 8 <= (int)blockIdx.x; t += 8) {
        uint32_t v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __ldg(col + (int64_t)(t + e) * bins);
#pragma unroll
        for (int e = 0; e < 8; ++e) before += v[e];
      }
      for (; t < (int)blockIdx.x; ++t) before += __ldg(col + (int64_t)t * bins);
      goff[b] = before;
      tsum += __ldg(dtot + b);
    }
    uint32_t dbase = block_exclusive_scan<kSortThreads>(tsum, ws, nullptr);
    for (int q = 0; q < per; ++q) {
      const int b = threadIdx.x * per + q;
      if (b >= bins) break;
      goff[b] += dbase; dbase += __ldg(dtot + b);
    }
  }
  __syncthreads();
  uint32_t* cnt = sh + warp * bins;
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base_i + r * 32 + lane;
    const bool ok = i < n;
    const unsigned act = __ballot_sync(0xffffffffu, ok);
    if (ok) {
      const uint32_t d = (key[r] >> shift) & (bins - 1);
      const unsigned m = __match_any_sync(act, d);
      const int leader = __ffs(m) - 1;
      uint32_t old = 0;
      if (lane == leader) { old = cnt[d]; cnt[d] = old + __popc(m); }
      old = __shfl_sync(m, old, leader);
      rnk[r] = old + __popc(m & ((1u << lane) - 1u));
    }
  }
  __syncthreads();
  // exclusive scan of the warp counts across warps, per digit, on top of the tile's global offset
  for (int b = threadIdx.x; b < bins; b += kSortThreads) {
    uint32_t run = goff[b];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) { const uint32_t c = sh[w * bins + b]; sh[w * bins + b] = run; run += c; }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base_i + r * 32 + lane;
    if (i < n) {
      const uint32_t d = (key[r] >> shift) & (bins - 1);
      const uint32_t dst = cnt[d] + rnk[r];
      out_key[dst] = key[r]; out_val[dst] = val[r];
    }
  }
}

struct SortBuffers { uint32_t *keyA, *valA, *keyB, *valB, *hist, *dtot; int tiles; };   // dtot: [passes][bins], zero on entry

inline int sort_tiles(int64_t n) { return (int)((n + kSortTile - 1) / kSortTile); }
inline size_t sort_hist_words(int tiles, int bits) { return (size_t)tiles * ((size_t)1 << bits) + 8; }
// per pass: digit totals + one row of digit sums per group of kSuperTile tiles
inline size_t sort_dtot_words_pass(int tiles, int bits) { return ((size_t)(1 + (tiles + kSuperTile - 1) / kSuperTile) << bits); }
inline size_t sort_dtot_words(int tiles, int bits, int passes) { return sort_dtot_words_pass(tiles, bits) * passes + 8; }

// Sorts positions 0..n-1 by key(src[p]) (stable); n is lowered to *n_dev when n_dev != nullptr.  bits*passes must cover the key range.  On return *skey / *spos point
// at the buffers holding the sorted keys and positions.  *dtot_out is the digit-total array of the LAST pass (its
// exclusive scan gives the first output index of each digit) or nullptr when the separate-scan path ran, in which case
// sb.hist holds the scanned digit-major histogram.  sb.dtot must be zero on entry.  *launches counts the kernels.
static int radix_sort_by_key(const int64_t* src, int64_t n, const int64_t* n_dev, int mod, int64_t cap, int bits, int passes, const SortBuffers& sb,
                             const uint32_t** skey, const uint32_t** spos, const uint32_t** dtot_out, int* launches, cudaStream_t st) {
  const size_t sm_hist = ((size_t)1 << bits) * 4, sm_scat = sm_hist * (kSortWarps + 1);
  if (sm_scat > 48 * 1024 &&
      note_cuda(cudaFuncSetAttribute(srm2_sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_scat)))
    return SRM2_ERR_CUDA;
  const int64_t entries = (int64_t)sb.tiles << bits;
  const bool separate_scan = entries > kFusedOffsetsLimit;
  uint32_t *ko = sb.keyA, *vo = sb.valA, *ki = nullptr, *vi = nullptr;
  uint32_t* dt = nullptr;
  for (int p = 0; p < passes; ++p) {
    const int shiftp = p * bits;
    dt = separate_scan ? nullptr : sb.dtot + sort_dtot_words_pass(sb.tiles, bits) * p;
    srm2_sort_hist_kernel<<<sb.tiles, kSortThreads, sm_hist, st>>>(p == 0 ? src : nullptr, ki, n, n_dev, shiftp, bits, sb.hist, dt, sb.tiles, cap, mod);
    if (separate_scan) {
      srm2_scan_exclusive_u32_kernel<<<1, kScanThreads, 0, st>>>(sb.hist, sb.hist, entries, nullptr, entries, 0, nullptr);
      *launches += 1;
    }
    srm2_sort_scatter_kernel<<<sb.tiles, kSortThreads, sm_scat, st>>>(p == 0 ? src : nullptr, ki, vi, n, n_dev, shiftp, bits, sb.hist, dt, sb.tiles,
                                                                     ko, vo, cap, mod);
    *launches += 2;
    ki = ko; vi = vo;
    ko = (ko == sb.keyA) ? sb.keyB : sb.keyA; vo = (vo == sb.valA) ? sb.valB : sb.valA;
  }
  *skey = ki; *spos = vi; *dtot_out = dt;
  return SRM2_OK;
}

}  // namespace srm2
