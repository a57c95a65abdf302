// Stable LSD radix sort of (32-bit key, lookup position) pairs, shared by the segment-reduce and the owner routing.
#pragma once
#include "common.cuh"
#include "scan.cuh"

namespace srm2 {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortRounds = 16;                              // elements per thread
constexpr int kSortTile = kSortThreads * kSortRounds;        // 4096 elements per CTA
constexpr int kMaxRadixBits = 11;

// Key of a 64-bit input value: mod == 0: the value itself, with anything outside [0, cap) mapped to `cap` (behind every
// real key); mod > 0: value mod `mod` (owner of a row id), negative values mapped to 0.
__device__ __forceinline__ uint32_t make_key(int64_t k, int64_t cap, int mod) {
  if (mod > 0) return k < 0 ? 0u : (uint32_t)(k % mod);
  return (k < 0 || k >= cap) ? (uint32_t)cap : (uint32_t)k;
}

// Histogram of one digit per tile; hist is digit-major: hist[d * tiles + tile].
// Pass 0 reads the keys from the int64 inverse array (key_lo == nullptr), later passes from the u32 ping-pong buffer.
static __global__ void __launch_bounds__(kSortThreads)
srm2_sort_hist_kernel(const int64_t* __restrict__ key64, const uint32_t* __restrict__ key32, int64_t n, int shift, int bits,
                      uint32_t* __restrict__ hist, int tiles, int64_t cap, int mod) {
  extern __shared__ uint32_t sh[];
  const int bins = 1 << bits;
  for (int b = threadIdx.x; b < bins; b += kSortThreads) sh[b] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kSortTile;
#pragma unroll 4
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < n) {
      const uint32_t k = key64 ? make_key(key64[i], cap, mod) : key32[i];
      atomicAdd(&sh[(k >> shift) & (bins - 1)], 1u);
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kSortThreads) hist[(int64_t)b * tiles + blockIdx.x] = sh[b];
}

// Stable scatter of one tile.  Warp w owns elements [w*512, (w+1)*512) of the tile and walks them in rounds of 32
// consecutive elements; __match_any_sync groups equal digits of a round, so the rank of an element among the equal
// digits of its warp's sub-range is (count so far) + (equal digits in lower lanes).  Warp counts are then scanned
// across the warps of the tile and added to the tile's global digit offset.
static __global__ void __launch_bounds__(kSortThreads)
srm2_sort_scatter_kernel(const int64_t* __restrict__ key64, const uint32_t* __restrict__ key32,
                         const uint32_t* __restrict__ val32, int64_t n, int shift, int bits,
                         const uint32_t* __restrict__ hist_scanned, int tiles, uint32_t* __restrict__ out_key,
                         uint32_t* __restrict__ out_val, int64_t cap, int mod) {
  extern __shared__ uint32_t sh[];                 // [kSortWarps][bins]
  const int bins = 1 << bits;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int b = threadIdx.x; b < bins * kSortWarps; b += kSortThreads) sh[b] = 0;
  __syncthreads();
  uint32_t* cnt = sh + warp * bins;
  const int64_t base = (int64_t)blockIdx.x * kSortTile + (int64_t)warp * (32 * kSortRounds);
  uint32_t key[kSortRounds], val[kSortRounds], rnk[kSortRounds];
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool ok = i < n;
    const unsigned act = __ballot_sync(0xffffffffu, ok);
    if (ok) {
      key[r] = key64 ? make_key(key64[i], cap, mod) : key32[i];
      val[r] = val32 ? val32[i] : (uint32_t)i;
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
  // exclusive scan of the warp counts across warps, per digit, plus the tile's global offset
  for (int b = threadIdx.x; b < bins; b += kSortThreads) {
    uint32_t run = hist_scanned[(int64_t)b * tiles + blockIdx.x];
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) { const uint32_t c = sh[w * bins + b]; sh[w * bins + b] = run; run += c; }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kSortRounds; ++r) {
    const int64_t i = base + r * 32 + lane;
    if (i < n) {
      const uint32_t d = (key[r] >> shift) & (bins - 1);
      const uint32_t dst = cnt[d] + rnk[r];
      out_key[dst] = key[r]; out_val[dst] = val[r];
    }
  }
}

struct SortBuffers { uint32_t *keyA, *valA, *keyB, *valB, *hist; int tiles; };

inline int sort_tiles(int64_t n) { return (int)((n + kSortTile - 1) / kSortTile); }

// Sorts positions 0..n-1 by key(src[p]) (stable).  bits*passes must cover the key range.  On return *skey / *spos point
// at the buffers holding the sorted keys and positions; sb.hist holds the scanned digit-major histogram of the LAST
// pass (hist[d * tiles] = first output index of digit d when passes == 1).  3 kernels per pass.
static int radix_sort_by_key(const int64_t* src, int64_t n, int mod, int64_t cap, int bits, int passes, const SortBuffers& sb,
                             const uint32_t** skey, const uint32_t** spos, cudaStream_t st) {
  const size_t sm_hist = ((size_t)1 << bits) * 4, sm_scat = sm_hist * kSortWarps;
  if (sm_scat > 48 * 1024 &&
      note_cuda(cudaFuncSetAttribute(srm2_sort_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_scat)))
    return SRM2_ERR_CUDA;
  uint32_t *ko = sb.keyA, *vo = sb.valA, *ki = nullptr, *vi = nullptr;
  for (int p = 0; p < passes; ++p) {
    const int shiftp = p * bits;
    srm2_sort_hist_kernel<<<sb.tiles, kSortThreads, sm_hist, st>>>(p == 0 ? src : nullptr, ki, n, shiftp, bits, sb.hist, sb.tiles, cap, mod);
    srm2_scan_exclusive_u32_kernel<<<1, kScanThreads, 0, st>>>(sb.hist, sb.hist, (int64_t)sb.tiles << bits, nullptr,
                                                               (int64_t)sb.tiles << bits, 0, nullptr);
    srm2_sort_scatter_kernel<<<sb.tiles, kSortThreads, sm_scat, st>>>(p == 0 ? src : nullptr, ki, vi, n, shiftp, bits, sb.hist,
                                                                     sb.tiles, ko, vo, cap, mod);
    ki = ko; vi = vo;
    ko = (ko == sb.keyA) ? sb.keyB : sb.keyA; vo = (vo == sb.valA) ? sb.valB : sb.valA;
  }
  *skey = ki; *spos = vi;
  return SRM2_OK;
}

}  // namespace srm2
