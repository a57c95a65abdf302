// Shared device/host helpers of the srm2_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "srm2_b200.h"

namespace srm2 {

// The B200 has 148 SMs; grids of the streaming kernels are sized in multiples of this.
constexpr int kSMs = 148;

// Grid of an index kernel (dedup, sort bookkeeping, segment boundaries, plans, requests, the exchange's kernels).  These
// kernels run beside the bandwidth-bound kernel of an earlier step, whose CTAs hold every register of every SM between
// them: a CTA of another kernel gets in when one of those retires, and for as long as it lives it takes that one's place.
// SM time is what the pipelined step runs out of, and an index kernel is bound by the latency of a few dependent loads,
// not by the number of its threads — so it gets a grid-stride loop on two CTAs per SM at most (the kernels that talk to
// other GPUs: one), which costs it little time and spends a fraction of the SM time of a grid sized by its input.
inline unsigned index_grid(int64_t blocks) {
  const int64_t cap = 2 * kSMs;
  return (unsigned)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

// Records a CUDA runtime error for srm2_last_cuda_error(); returns SRM2_ERR_CUDA or SRM2_OK.
int note_cuda(cudaError_t e);

// Kernel-launch bookkeeping for srm2_launch_count(): k kernels were just enqueued.
void add_launches(int k);
inline int launch_status(int k = 1) { add_launches(k); return note_cuda(cudaGetLastError()); }

// Optional instrumentation (srm2_stage_events): events recorded around the gradient-streaming stage of a pipeline.
void stage_begin(cudaStream_t st);
void stage_end(cudaStream_t st);

// Effective element count of a kernel: the host bound, lowered by an optional device-resident count.
__device__ __forceinline__ int64_t eff_count(int64_t n_host, const int64_t* n_dev) {
  if (n_dev == nullptr) return n_host;
  const int64_t v = *n_dev;
  return v < 0 ? 0 : (v < n_host ? v : n_host);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- exact fp32 arithmetic: every operation rounded on its own, never contracted ----------------
struct AdamSc { float lr, b1, omb1, b2, omb2, bc1, bc2, eps; };

// One Adam step on one element, in the operation order of the reference
// (srm2/ops.py:50-56 == srm2/csrc/srm2_cpu.cpp:27-32).
__device__ __forceinline__ void adam_elem(float& w, float& m, float& v, float g, const AdamSc& s) {
  m = __fadd_rn(__fmul_rn(s.b1, m), __fmul_rn(s.omb1, g));
  const float t2 = __fmul_rn(s.omb2, g);
  v = __fadd_rn(__fmul_rn(s.b2, v), __fmul_rn(t2, g));
  const float mh = __fdiv_rn(m, s.bc1);
  const float vh = __fdiv_rn(v, s.bc2);
  const float den = __fadd_rn(__fsqrt_rn(vh), s.eps);
  w = __fsub_rn(w, __fdiv_rn(__fmul_rn(s.lr, mh), den));
}

__device__ __forceinline__ void adam_vec4(float4& w, float4& m, float4& v, const float4& g, const AdamSc& s) {
  adam_elem(w.x, m.x, v.x, g.x, s);
  adam_elem(w.y, m.y, v.y, g.y, s);
  adam_elem(w.z, m.z, v.z, g.z, s);
  adam_elem(w.w, m.w, v.w, g.w, s);
}

// murmur3 fmix32 (srm2/gpu_ops.py:15-23)
__device__ __forceinline__ uint32_t fmix32(uint32_t x) {
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

// Initial weight of element j of row r (srm2/gpu_ops.py:29-34).  rowkey = fmix32((uint32)(r>>32) + seed),
// base = (uint32)(r*D).  u*2-1 is exact; the product with bound is the single rounding.
__device__ __forceinline__ float init_elem(uint32_t base, uint32_t j, uint32_t rowkey, uint32_t seed, float bound) {
  const uint32_t h = fmix32(((base + j) ^ rowkey) ^ seed);
  const float u = __fmul_rn(__uint2float_rn(h >> 8), 1.0f / 16777216.0f);
  return __fmul_rn(__fsub_rn(__fmul_rn(u, 2.0f), 1.0f), bound);
}

// streaming (read-once) 16-byte load / store
__device__ __forceinline__ float4 ld_stream4(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st_stream4(float* p, const float4& v) { __stcs(reinterpret_cast<float4*>(p), v); }

}  // namespace srm2
