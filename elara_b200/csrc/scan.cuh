// Block-level scan helpers and a single-CTA exclusive scan kernel for the small integer arrays
// (histograms, per-segment counts) that the dedup / sort / segment kernels produce.
#pragma once
#include "common.cuh"

namespace srm2 {

constexpr int kScanThreads = 1024;

// Exclusive scan of one value per thread over a block of NT threads (NT multiple of 32, <= 1024).
// Returns the exclusive prefix of `v`; *total (optional) receives the block sum.  `ws` is 33 words of shared memory.
template <int NT>
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* ws, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) ws[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t s = lane < NT / 32 ? ws[lane] : 0u;
    uint32_t si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += t;
    }
    ws[lane] = si - s;                 // exclusive prefix of the warp sums
    if (lane == 31) ws[32] = si;       // block total
  }
  __syncthreads();
  const uint32_t res = ws[warp] + inc - v;
  if (total) *total = ws[32];
  __syncthreads();                     // ws may be reused by the caller
  return res;
}

// The same for a 64-bit value (three counters packed into one word scan together).  `ws` is 33 64-bit words.
template <int NT>
__device__ __forceinline__ uint64_t block_exclusive_scan64(uint64_t v, uint64_t* ws, uint64_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint64_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint64_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) ws[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint64_t s = lane < NT / 32 ? ws[lane] : 0ull;
    uint64_t si = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint64_t t = __shfl_up_sync(0xffffffffu, si, o);
      if (lane >= o) si += t;
    }
    ws[lane] = si - s;
    if (lane == 31) ws[32] = si;
  }
  __syncthreads();
  const uint64_t res = ws[warp] + inc - v;
  if (total) *total = ws[32];
  __syncthreads();
  return res;
}

// out[i] = sum_{k<i} in[i]  for i < count (count read from *count_dev when count_dev != nullptr, else count_host);
// count is clamped to count_cap (the allocated length); optionally out[count] = total and *total_out = total.  One CTA of kScanThreads threads.
// in == out is allowed (and used by the sort): the two pointers are therefore not declared __restrict__.
static __global__ void __launch_bounds__(kScanThreads)
srm2_scan_exclusive_u32_kernel(const uint32_t* in, uint32_t* out, int64_t count_host,
                               const int64_t* __restrict__ count_dev, int64_t count_cap, int write_tail,
                               uint32_t* __restrict__ total_out) {
  __shared__ uint32_t ws[33];
  int64_t count = count_dev ? *count_dev : count_host;
  if (count > count_cap) count = count_cap;
  // rounds of 4 * kScanThreads consecutive entries; thread t owns entries [4t, 4t+4) of the round (coalesced)
  uint32_t carry = 0;
  for (int64_t base = 0; base < count; base += 4 * kScanThreads) {
    const int64_t i0 = base + 4 * (int64_t)threadIdx.x;
    uint32_t x[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = (i0 + e < count) ? in[i0 + e] : 0u;
    uint32_t tot;
    uint32_t run = carry + block_exclusive_scan<kScanThreads>(x[0] + x[1] + x[2] + x[3], ws, &tot);
#pragma unroll
    for (int e = 0; e < 4; ++e) { if (i0 + e < count) out[i0 + e] = run; run += x[e]; }
    carry += tot;
  }
  const uint32_t total = carry;
  if (threadIdx.x == 0) {
    if (write_tail) out[count] = total;
    if (total_out) *total_out = total;
  }
}

}  // namespace srm2
