// Counter-hash row initialisation and exact replay of logged gradients.
//
// Both kernels write one [3,D] record per requested row and never read the tables: init is write-only
// (3*D*4 bytes per row), replay additionally streams cnt gradient rows of D*4 bytes from the flat log.
// Work item = one 16-byte lane (row i, quarter-vector j4), consecutive threads = consecutive lanes, so a
// row's D/4 threads write three fully used D*4-byte runs.  Outputs are written once and not re-read by
// these kernels, hence streaming stores.  Bound by HBM bandwidth.
#include "common.cuh"
#include "exact.cuh"

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
      adam_vec4_fast(w, m, v, g[k], adam_fast_prepare(sc));
    }
  }
  float* b = out + i * 3 * D + j4 * 4;
  st_stream4(b, w); st_stream4(b + D, m); st_stream4(b + 2 * D, v);
}

// ---- replay as a software pipeline -------------------------------------------------------------------------------------
// Persistent CTAs walk the (row, 16-byte lane) items with a grid stride.  Every thread stages the logged gradients of its
// NEXT item in its own shared-memory slots with cp.async (no registers held, no instruction issued while they fly) and
// fetches the row descriptors (row id, offset, count, steps) of the item after that, while it runs the arithmetic of the
// current item; cp.async.wait_group 1 is the only wait, and a thread only reads back what it copied itself.
// The per-step scalars — each in both lanes of a register pair, the reciprocals of the bias corrections and the range
// flag (exact.cuh) — are prepared once per CTA for every row of the scalar table and kept in shared memory, so a logged
// entry costs six 16-byte shared loads instead of two global loads, two reciprocals and the range checks per thread.
constexpr int kRpThreads = 256;
constexpr int kRpMaxTableRows = 384;                   // 36 KB of prepared scalars at most

__device__ __forceinline__ void rp_cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}

template <int KMAX, int MINB>
__global__ void __launch_bounds__(kRpThreads, MINB)
srm2_replay_rows_pipelined_kernel(float* __restrict__ out, const int64_t* __restrict__ rows, const float* __restrict__ logs,
                                  const int64_t* __restrict__ offs, const int32_t* __restrict__ steps,
                                  const int32_t* __restrict__ cnt, uint32_t n, int shift, int D, int K,
                                  uint32_t seed, float bound, const float* __restrict__ table, int table_rows) {
  extern __shared__ __align__(16) unsigned char rp_smem[];
  float4* stage = reinterpret_cast<float4*>(rp_smem);                                   // [2][KMAX][kRpThreads]
  AdamFast* prep = reinterpret_cast<AdamFast*>(rp_smem + 2 * KMAX * kRpThreads * 16);  // [table_rows]
  for (int r = threadIdx.x; r < table_rows; r += kRpThreads) prep[r] = adam_fast_prepare(load_sc(table, table_rows, r));
  __syncthreads();
  const ExactConst ec = exact_const();
  const pf2 bound2 = pk1(bound);
  // rows advance by a fixed number per iteration; the 16-byte lane of a thread never changes
  const uint32_t t0 = blockIdx.x * kRpThreads + threadIdx.x;
  const uint32_t j = (t0 & ((1u << shift) - 1u)) * 4u;                    // first element of this thread's lane
  const uint32_t rstep = (gridDim.x * kRpThreads) >> shift;
  uint32_t i = t0 >> shift;
  const float* logs_j = logs + j;
  float* out_j = out + j;
  const uint32_t rec = 3u * (uint32_t)D;
  const unsigned s_mine = (unsigned)__cvta_generic_to_shared(stage + threadIdx.x);
  constexpr unsigned kSlot = kRpThreads * 16, kBuf = KMAX * kSlot;

  // what a thread keeps per row: for the copies (source address, entry count) and for the arithmetic (hash inputs, steps)
  auto load_copy = [&](uint32_t ii, const float*& src, int& c) {
    c = 0; src = logs_j;
    if (ii < n) { const int cc = __ldg(cnt + ii); c = cc < 0 ? 0 : (cc > K ? K : cc); src = logs_j + __ldg(offs + ii) * D; }
  };
  auto load_hash = [&](uint32_t ii, uint32_t& rowkey, uint32_t& base, int (&st)[KMAX]) {
    rowkey = 0; base = 0;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) st[k] = 0;
    if (ii < n) {
      const uint64_t r = (uint64_t)__ldg(rows + ii);
      rowkey = fmix32((uint32_t)(r >> 32) + seed); base = (uint32_t)r * (uint32_t)D + j;
      const int32_t* sp = steps + (size_t)ii * K;
#pragma unroll
      for (int k = 0; k < KMAX; ++k) if (k < K) st[k] = __ldg(sp + k);
    }
  };
  auto issue = [&](const float* src, int c, unsigned sbuf) {
#pragma unroll
    for (int k = 0; k < KMAX; ++k) {
      if (k < c) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s_mine + sbuf + k * kSlot), "l"(src) : "memory");
      src += D;
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };

  const float* src_n; int c_cur, c_n;                       // copies: the next row's
  uint32_t rowkey, base, rowkey_n, base_n; int st[KMAX], st_n[KMAX];
  load_copy(i, src_n, c_cur);
  load_hash(i, rowkey, base, st);
  unsigned sbuf = 0;
  issue(src_n, c_cur, 0);
  load_copy(i + rstep, src_n, c_n);
  for (; i < n; i += rstep) {
    issue(src_n, c_n, sbuf ^ kBuf);                         // gradients of the next row
    const int c_nn_owner = c_n;
    load_hash(i + rstep, rowkey_n, base_n, st_n);           // used by the next iteration
    load_copy(i + 2 * rstep, src_n, c_n);                   // used at the top of the next iteration
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    Quad w = Quad{init_pair(base, 0, rowkey, seed, bound2), init_pair(base, 2, rowkey, seed, bound2)};
    Quad m = Quad{pk1(0.f), pk1(0.f)}, v = m;
    unsigned sg = s_mine + sbuf;
#pragma unroll 1
    for (int k = 0; k < c_cur; ++k) {                       // a rolled loop: w, m, v stay in place, the steps rotate through st[0]
      const int s0 = st[0];
#pragma unroll
      for (int q = 0; q + 1 < KMAX; ++q) st[q] = st[q + 1];
      const AdamFast f = prep[(unsigned)s0 < (unsigned)table_rows ? s0 : 0];
      float4 g;
      asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(g.x), "=f"(g.y), "=f"(g.z), "=f"(g.w) : "r"(sg));
      adam_quad_fast(w, m, v, quad(g), f, ec);
      sg += kSlot;
    }
    float* b = out_j + (size_t)i * rec;
    st_stream4(b, unquad(w)); st_stream4(b + D, unquad(m)); st_stream4(b + 2 * D, unquad(v));
    c_cur = c_nn_owner; rowkey = rowkey_n; base = base_n;
#pragma unroll
    for (int k = 0; k < KMAX; ++k) st[k] = st_n[k];
    sbuf ^= kBuf;
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
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
    if (shift >= 0 && lpr <= kRpThreads && K <= 4 && table_rows <= kRpMaxTableRows && n < ((int64_t)1 << 31) - (int64_t)kSMs * 5 * 3 * kRpThreads) {
      // K <= 3 (the reference's default history depth): three staging slots per buffer
      const int km = K <= 3 ? 3 : 4, minb = 4;
      const size_t smem = (size_t)2 * km * kRpThreads * 16 + (size_t)table_rows * sizeof(AdamFast);
      const int64_t grid = blocks < (int64_t)kSMs * minb ? blocks : (int64_t)kSMs * minb;
      if (K <= 3) {
        if (note_cuda(cudaFuncSetAttribute(srm2_replay_rows_pipelined_kernel<3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem))) return SRM2_ERR_CUDA;
        srm2_replay_rows_pipelined_kernel<3, 4><<<(unsigned)grid, kRpThreads, smem, st>>>(out, rows, logs, offs, steps, cnt, (uint32_t)n, shift, (int)D,
                                                                                       (int)K, seed, bound, table, (int)table_rows);
      } else {
        if (note_cuda(cudaFuncSetAttribute(srm2_replay_rows_pipelined_kernel<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem))) return SRM2_ERR_CUDA;
        srm2_replay_rows_pipelined_kernel<4, 4><<<(unsigned)grid, kRpThreads, smem, st>>>(out, rows, logs, offs, steps, cnt, (uint32_t)n, shift, (int)D,
                                                                                       (int)K, seed, bound, table, (int)table_rows);
      }
    } else if (K <= 4)
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
