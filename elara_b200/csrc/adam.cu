// Row-sparse Adam over an interleaved [C,3,D] fp32 pool (w, m, v per row).
//
// Work decomposition: one "item" is one 16-byte quarter-vector position (row i, lane j4) — a thread reads
// the float4 of w, m, v and g at that position, applies Adam to its four elements and writes w, m, v
// back.  Consecutive threads own consecutive positions, so the D/4 threads of a row read three fully
// used D*4-byte runs of the pool and one run of the gradient matrix (which, being [n,D] contiguous, is
// read as one linear float4 stream).  The kernel is a pure gather/update/scatter: 7*D*4 bytes of HBM
// traffic per row plus the slot index, no reuse, so it is bound by HBM bandwidth; each thread keeps
// U*4 independent 16-byte loads in flight.
#include "common.cuh"
#include "exact.cuh"

namespace srm2 {

constexpr int kAdamThreads = 256;

template <typename SlotT, int U>
__global__ void __launch_bounds__(kAdamThreads)
srm2_adam_rows_kernel(float* __restrict__ pool, const SlotT* __restrict__ slots, const float* __restrict__ grad,
                      int64_t items, int lpr, int shift, int64_t rec, int D, AdamSc sc) {
  const int64_t t0 = (int64_t)blockIdx.x * (kAdamThreads * U) + threadIdx.x;
  float4 w[U], m[U], v[U], g[U];
  float* base[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t t = t0 + (int64_t)u * kAdamThreads;
    base[u] = nullptr;
    if (t < items) {
      int64_t i; int j4;
      if (shift >= 0) { i = t >> shift; j4 = (int)(t & (lpr - 1)); } else { i = t / lpr; j4 = (int)(t - i * lpr); }
      const int64_t slot = (int64_t)slots[i];
      float* b = pool + slot * rec + j4 * 4;
      base[u] = b;
      g[u] = ld_stream4(grad + t * 4);
      w[u] = *reinterpret_cast<const float4*>(b);
      m[u] = *reinterpret_cast<const float4*>(b + D);
      v[u] = *reinterpret_cast<const float4*>(b + 2 * D);
    }
  }
  const AdamFast fa = adam_fast_prepare(sc);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (base[u] != nullptr) {
      adam_vec4_fast(w[u], m[u], v[u], g[u], fa);
      *reinterpret_cast<float4*>(base[u]) = w[u];
      *reinterpret_cast<float4*>(base[u] + D) = m[u];
      *reinterpret_cast<float4*>(base[u] + 2 * D) = v[u];
    }
  }
}

// Any D, any alignment: one element per thread.
template <typename SlotT>
__global__ void __launch_bounds__(kAdamThreads)
srm2_adam_rows_scalar_kernel(float* __restrict__ pool, const SlotT* __restrict__ slots, const float* __restrict__ grad,
                             int64_t items, int D, AdamSc sc) {
  const int64_t t = (int64_t)blockIdx.x * kAdamThreads + threadIdx.x;
  if (t >= items) return;
  const int64_t i = t / D; const int j = (int)(t - i * D);
  float* b = pool + (int64_t)slots[i] * 3 * D + j;
  float w = b[0], m = b[D], v = b[2 * D];
  adam_elem(w, m, v, grad[t], sc);
  b[0] = w; b[D] = m; b[2 * D] = v;
}

template <typename SlotT>
static int launch_adam(float* pool, const SlotT* slots, const float* grad, int64_t n, int64_t D, const AdamSc& sc,
                       cudaStream_t st) {
  if ((D & 3) == 0 && aligned16(pool) && aligned16(grad)) {
    const int lpr = (int)(D / 4);
    const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
    const int64_t items = n * lpr;
    constexpr int U = 2;
    const int64_t blocks = (items + kAdamThreads * U - 1) / (kAdamThreads * U);
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    srm2_adam_rows_kernel<SlotT, U><<<(unsigned)blocks, kAdamThreads, 0, st>>>(pool, slots, grad, items, lpr, shift,
                                                                             3 * D, (int)D, sc);
  } else {
    const int64_t items = n * D;
    const int64_t blocks = (items + kAdamThreads - 1) / kAdamThreads;
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    srm2_adam_rows_scalar_kernel<SlotT><<<(unsigned)blocks, kAdamThreads, 0, st>>>(pool, slots, grad, items, (int)D, sc);
  }
  return launch_status();
}

}  // namespace srm2

extern "C" int srm2_adam_rows_f32(float* pool, const void* slots, int slots_is_i64, const float* grad, int64_t n,
                                  int64_t D, const float sc[8], srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0 || sc == nullptr) return SRM2_ERR_ARG;
  if (n == 0) return SRM2_OK;
  if (pool == nullptr || slots == nullptr || grad == nullptr) return SRM2_ERR_ARG;
  if (D > (1 << 20)) return SRM2_ERR_UNSUPPORTED;
  const AdamSc s{sc[0], sc[1], sc[2], sc[3], sc[4], sc[5], sc[6], sc[7]};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return slots_is_i64 ? launch_adam<int64_t>(pool, static_cast<const int64_t*>(slots), grad, n, D, s, st)
                      : launch_adam<int32_t>(pool, static_cast<const int32_t*>(slots), grad, n, D, s, st);
}
