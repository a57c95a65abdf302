// Counter-hash row initialisation and exact replay of logged gradients.
//
// Both kernels write one [3,D] record per requested row and never read the tables: init is write-only
// (3*D*4 bytes per row), replay additionally streams cnt gradient rows of D*4 bytes from the flat log.
// Work item = one 16-byte lane (row i, quarter-vector j4), consecutive threads = consecutive lanes, so a
// row's D/4 threads write three fully used D*4-byte runs.  Outputs are written once and not re-read by
// these kernels, hence streaming stores.  Bound by HBM bandwidth.
#include "common.cuh"

namespace srm2 {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
srm2_init_rows_kernel(float* __restrict__ out, const int64_t* __restrict__ rows, int64_t items, int lpr, int shift,
                      int D, uint32_t seed, float bound) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= items) return;
  int64_t i; int j4;
  if (shift >= 0) { i = t >> shift; j4 = (int)(t & (lpr - 1)); } else { i = t / lpr; j4 = (int)(t - i * lpr); }
  const int64_t r = rows[i];
  const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + seed);
  const uint32_t base = (uint32_t)(uint64_t)r * (uint32_t)D + (uint32_t)(j4 * 4);
  float4 w;
  w.x = init_elem(base, 0, rowkey, seed, bound);
  w.y = init_elem(base, 1, rowkey, seed, bound);
  w.z = init_elem(base, 2, rowkey, seed, bound);
  w.w = init_elem(base, 3, rowkey, seed, bound);
  float* b = out + i * 3 * D + j4 * 4;
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  st_stream4(b, w); st_stream4(b + D, z); st_stream4(b + 2 * D, z);
}

__global__ void __launch_bounds__(kThreads)
srm2_init_rows_scalar_kernel(float* __restrict__ out, const int64_t* __restrict__ rows, int64_t items, int D,
                             uint32_t seed, float bound) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= items) return;
  const int64_t i = t / D; const int j = (int)(t - i * D);
  const int64_t r = rows[i];
  const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + seed);
  float* b = out + i * 3 * D + j;
  b[0] = init_elem((uint32_t)(uint64_t)r * (uint32_t)D, (uint32_t)j, rowkey, seed, bound);
  b[D] = 0.f; b[2 * D] = 0.f;
}

// Scalars of one logical step; steps outside the table read row 0 (all zeros, which turns the row into
// NaNs instead of reading out of bounds).
__device__ __forceinline__ AdamSc load_sc(const float* __restrict__ table, int64_t table_rows, int step) {
  const int64_t s = (step >= 0 && step < table_rows) ? step : 0;
  const float4 a = __ldg(reinterpret_cast<const float4*>(table + s * 8));
  const float4 b = __ldg(reinterpret_cast<const float4*>(table + s * 8 + 4));
  return AdamSc{a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
}

template <int KMAX>
__global__ void __launch_bounds__(kThreads)
srm2_replay_rows_kernel(float* __restrict__ out, const int64_t* __restrict__ rows, const float* __restrict__ logs,
                        const int64_t* __restrict__ offs, const int32_t* __restrict__ steps,
                        const int32_t* __restrict__ cnt, int64_t items, int lpr, int shift, int D, int K,
                        uint32_t seed, float bound, const float* __restrict__ table, int64_t table_rows) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= items) return;
  int64_t i; int j4;
  if (shift >= 0) { i = t >> shift; j4 = (int)(t & (lpr - 1)); } else { i = t / lpr; j4 = (int)(t - i * lpr); }
  const int64_t r = rows[i];
  int c = cnt[i]; c = c < 0 ? 0 : (c > K ? K : c);
  const int64_t o = offs[i];
  // issue every gradient load before any arithmetic
  float4 g[KMAX]; int st[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    if (k < c) {
      g[k] = ld_stream4(logs + (o + k) * D + j4 * 4);
      st[k] = steps[i * K + k];
    }
  }
  const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + seed);
  const uint32_t base = (uint32_t)(uint64_t)r * (uint32_t)D + (uint32_t)(j4 * 4);
  float4 w, m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
  w.x = init_elem(base, 0, rowkey, seed, bound);
  w.y = init_elem(base, 1, rowkey, seed, bound);
  w.z = init_elem(base, 2, rowkey, seed, bound);
  w.w = init_elem(base, 3, rowkey, seed, bound);
#pragma unroll
  for (int k = 0; k < KMAX; ++k) {
    if (k < c) {
      const AdamSc sc = load_sc(table, table_rows, st[k]);
      adam_vec4(w, m, v, g[k], sc);
    }
  }
  float* b = out + i * 3 * D + j4 * 4;
  st_stream4(b, w); st_stream4(b + D, m); st_stream4(b + 2 * D, v);
}

// Any D, K and alignment: one element per thread, entries applied in a plain loop.
__global__ void __launch_bounds__(kThreads)
srm2_replay_rows_scalar_kernel(float* __restrict__ out, const int64_t* __restrict__ rows, const float* __restrict__ logs,
                               const int64_t* __restrict__ offs, const int32_t* __restrict__ steps,
                               const int32_t* __restrict__ cnt, int64_t items, int D, int K, uint32_t seed, float bound,
                               const float* __restrict__ table, int64_t table_rows) {
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= items) return;
  const int64_t i = t / D; const int j = (int)(t - i * D);
  const int64_t r = rows[i];
  int c = cnt[i]; c = c < 0 ? 0 : (c > K ? K : c);
  const int64_t o = offs[i];
  const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + seed);
  float w = init_elem((uint32_t)(uint64_t)r * (uint32_t)D, (uint32_t)j, rowkey, seed, bound), m = 0.f, v = 0.f;
  for (int k = 0; k < c; ++k) {
    const int s0 = steps[i * K + k];
    const int64_t s = (s0 >= 0 && s0 < table_rows) ? s0 : 0;
    const float* p = table + s * 8;
    const AdamSc sc{__ldg(p), __ldg(p + 1), __ldg(p + 2), __ldg(p + 3), __ldg(p + 4), __ldg(p + 5), __ldg(p + 6), __ldg(p + 7)};
    adam_elem(w, m, v, logs[(o + k) * D + j], sc);
  }
  float* b = out + i * 3 * D + j;
  b[0] = w; b[D] = m; b[2 * D] = v;
}

}  // namespace srm2

extern "C" int srm2_init_rows_f32(float* out, const int64_t* rows, int64_t n, int64_t D, uint32_t seed, float bound,
                                  srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0) return SRM2_ERR_ARG;
  if (n == 0) return SRM2_OK;
  if (out == nullptr || rows == nullptr) return SRM2_ERR_ARG;
  if (D > (1 << 20)) return SRM2_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((D & 3) == 0 && aligned16(out)) {
    const int lpr = (int)(D / 4);
    const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
    const int64_t items = n * lpr, blocks = (items + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    srm2_init_rows_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(out, rows, items, lpr, shift, (int)D, seed, bound);
  } else {
    const int64_t items = n * D, blocks = (items + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    srm2_init_rows_scalar_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(out, rows, items, (int)D, seed, bound);
  }
  return launch_status();
}

extern "C" int srm2_replay_rows_f32(float* out, const int64_t* rows, const float* logs, const int64_t* offs,
                                    const int32_t* steps, const int32_t* cnt, int64_t n, int64_t D, int64_t K,
                                    uint32_t seed, float bound, const float* table, int64_t table_rows,
                                    srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0 || K < 0 || table_rows < 1) return SRM2_ERR_ARG;
  if (n == 0) return SRM2_OK;
  if (out == nullptr || rows == nullptr || offs == nullptr || cnt == nullptr || table == nullptr) return SRM2_ERR_ARG;
  if (K > 0 && (steps == nullptr || logs == nullptr)) return SRM2_ERR_ARG;
  if (D > (1 << 20) || K > (1 << 20)) return SRM2_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = (D & 3) == 0 && aligned16(out) && (logs == nullptr || aligned16(logs)) && aligned16(table) && K <= 8;
  if (vec) {
    const int lpr = (int)(D / 4);
    const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
    const int64_t items = n * lpr, blocks = (items + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    if (K <= 4)
      srm2_replay_rows_kernel<4><<<(unsigned)blocks, kThreads, 0, st>>>(out, rows, logs, offs, steps, cnt, items, lpr, shift,
                                                                       (int)D, (int)K, seed, bound, table, table_rows);
    else
      srm2_replay_rows_kernel<8><<<(unsigned)blocks, kThreads, 0, st>>>(out, rows, logs, offs, steps, cnt, items, lpr, shift,
                                                                       (int)D, (int)K, seed, bound, table, table_rows);
  } else {
    const int64_t items = n * D, blocks = (items + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
    srm2_replay_rows_scalar_kernel<<<(unsigned)blocks, kThreads, 0, st>>>(out, rows, logs, offs, steps, cnt, items, (int)D,
                                                                         (int)K, seed, bound, table, table_rows);
  }
  return launch_status();
}
