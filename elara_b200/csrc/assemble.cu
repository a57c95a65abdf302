// Fused assemble: the working matrix W [n, D] of a step — one weight row per unique row of the batch — built by one
// kernel from its five sources (srm2/elara.py:471-489 does this with init_rows, replay_rows and ten index ops):
//   resident rows      W[hit_pos[i]] = pool[hit_slot[i], 0]
//   never-touched rows fullN[i] = counter-hash init of N_row[i];                W[N_pos[i]] = fullN[i, 0]
//   logged rows        fullL[i] = replay of L_row[i]'s <= K logged gradients;   W[L_pos[i]] = fullL[i, 0]
//   staged full rows   W[F_pos[i]] = ff[i, 0]
//   staged weights     W[S_pos[i]] = sw[i]
// fullN and fullL are kept: the update step scatters them into the pool.  One thread per 16-byte lane of one source row;
// the five sources are consecutive ranges of the item space, so a warp rarely spans two of them.  Arithmetic of the
// init and replay rows is the same code as the standalone kernels (common.cuh), hence the same bits.
#include "common.cuh"
#include "exact.cuh"

namespace srm2 {

struct AssembleArgs {
  float* W; int D; int lpr; int shift; int K;
  const float* pool; const int64_t* hit_pos; const int64_t* hit_slot;
  float* fullN; const int64_t* N_pos; const int64_t* N_row; uint32_t seed; float bound;
  float* fullL; const int64_t* L_pos; const int64_t* L_row; const float* logs; const int64_t* L_off; const int32_t* L_steps; const int32_t* L_cnt;
  const float* table; int64_t table_rows;
  const float* ff; const int64_t* F_pos;
  const float* sw; const int64_t* S_pos;
  int64_t end_hit, end_N, end_L, end_F, end_S;       // exclusive ends of the five item ranges (in 16-byte lanes)
  int64_t n;                                         // rows of W
};

__device__ __forceinline__ AdamSc assemble_sc(const float* __restrict__ table, int64_t table_rows, int step) {
  const int64_t s = (step >= 0 && step < table_rows) ? step : 0;      // as the replay kernel: row 0 for a bad step
  const float4 a = __ldg(reinterpret_cast<const float4*>(table + s * 8));
  const float4 b = __ldg(reinterpret_cast<const float4*>(table + s * 8 + 4));
  return AdamSc{a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
}

template <int KMAX>
__global__ void __launch_bounds__(256)
srm2_assemble_kernel(AssembleArgs a) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= a.end_S) return;
  auto split = [&](int64_t tt, int64_t& i, int& j4) {
    if (a.shift >= 0) { i = tt >> a.shift; j4 = (int)(tt & (a.lpr - 1)); } else { i = tt / a.lpr; j4 = (int)(tt - i * a.lpr); }
  };
  auto put = [&](int64_t pos, int j4, const float4& w) {
    if (pos >= 0 && pos < a.n) *reinterpret_cast<float4*>(a.W + pos * a.D + j4 * 4) = w;     // a bad position is skipped
  };
  int64_t i; int j4;
  const int D = a.D;
  if (t < a.end_hit) {
    split(t, i, j4);
    put(a.hit_pos[i], j4, __ldg(reinterpret_cast<const float4*>(a.pool + a.hit_slot[i] * (3 * (int64_t)D) + j4 * 4)));
  } else if (t < a.end_N) {
    split(t - a.end_hit, i, j4);
    const int64_t r = a.N_row[i];
    const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + a.seed);
    const uint32_t base = (uint32_t)(uint64_t)r * (uint32_t)D + (uint32_t)(j4 * 4);
    float4 w;
    w.x = init_elem(base, 0, rowkey, a.seed, a.bound); w.y = init_elem(base, 1, rowkey, a.seed, a.bound);
    w.z = init_elem(base, 2, rowkey, a.seed, a.bound); w.w = init_elem(base, 3, rowkey, a.seed, a.bound);
    float* b = a.fullN + i * 3 * D + j4 * 4;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    st_stream4(b, w); st_stream4(b + D, z); st_stream4(b + 2 * D, z);
    put(a.N_pos[i], j4, w);
  } else if (t < a.end_L) {
    split(t - a.end_N, i, j4);
    const int64_t r = a.L_row[i];
    int c = a.L_cnt[i]; c = c < 0 ? 0 : (c > a.K ? a.K : c);
    const int64_t o = a.L_off[i];
    float4 g[KMAX]; int st[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k)
      if (k < c) { g[k] = ld_stream4(a.logs + (o + k) * D + j4 * 4); st[k] = a.L_steps[i * a.K + k]; }
    const uint32_t rowkey = fmix32((uint32_t)((uint64_t)r >> 32) + a.seed);
    const uint32_t base = (uint32_t)(uint64_t)r * (uint32_t)D + (uint32_t)(j4 * 4);
    float4 w, m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
    w.x = init_elem(base, 0, rowkey, a.seed, a.bound); w.y = init_elem(base, 1, rowkey, a.seed, a.bound);
    w.z = init_elem(base, 2, rowkey, a.seed, a.bound); w.w = init_elem(base, 3, rowkey, a.seed, a.bound);
#pragma unroll
    for (int k = 0; k < KMAX; ++k)
      if (k < c) { const AdamSc sc = assemble_sc(a.table, a.table_rows, st[k]); adam_vec4_fast(w, m, v, g[k], adam_fast_prepare(sc)); }
    float* b = a.fullL + i * 3 * D + j4 * 4;
    st_stream4(b, w); st_stream4(b + D, m); st_stream4(b + 2 * D, v);
    put(a.L_pos[i], j4, w);
  } else if (t < a.end_F) {
    split(t - a.end_L, i, j4);
    put(a.F_pos[i], j4, ld_stream4(a.ff + i * 3 * D + j4 * 4));
  } else {
    split(t - a.end_F, i, j4);
    put(a.S_pos[i], j4, ld_stream4(a.sw + i * D + j4 * 4));
  }
}

// Forward gather of the step: emb[p] = W[inv[p]] (srm2/train.py:427).  W has just been written by the assemble kernel and
// sits in L2 (n_unique x D x 4 bytes, ~25 MB for a DLRM-shaped step), so the lookups' rows are served from there: the
// gather writes n*D*4 bytes to HBM and reads almost nothing from it.
__global__ void __launch_bounds__(256)
srm2_gather_rows_kernel(float* __restrict__ out, const float* __restrict__ W, const int64_t* __restrict__ inv, int64_t items, int lpr,
                        int shift, int D, int64_t n_rows) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= items) return;
  int64_t p; int j4;
  if (shift >= 0) { p = t >> shift; j4 = (int)(t & (lpr - 1)); } else { p = t / lpr; j4 = (int)(t - p * lpr); }
  const int64_t r = inv[p];
  const float4 v = (r >= 0 && r < n_rows) ? *reinterpret_cast<const float4*>(W + r * D + j4 * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
  st_stream4(out + p * D + j4 * 4, v);
}

}  // namespace srm2

extern "C" int srm2_gather_rows_f32(float* out, const float* W, const int64_t* inv, int64_t n, int64_t n_rows, int64_t D, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || n_rows < 0 || D <= 0) return SRM2_ERR_ARG;
  if (n == 0) return SRM2_OK;
  if (out == nullptr || W == nullptr || inv == nullptr) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || !aligned16(out) || !aligned16(W)) return SRM2_ERR_UNSUPPORTED;
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  const int64_t items = n * lpr, blocks = (items + 255) / 256;
  if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
  srm2_gather_rows_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(out, W, inv, items, lpr, shift, (int)D, n_rows);
  return launch_status();
}

extern "C" int srm2_assemble_f32(float* W, int64_t n, int64_t D, const float* pool, const int64_t* hit_pos, const int64_t* hit_slot,
                                 int64_t n_hit, float* fullN, const int64_t* N_pos, const int64_t* N_row, int64_t n_N, uint32_t seed,
                                 float bound, float* fullL, const int64_t* L_pos, const int64_t* L_row, const float* logs,
                                 const int64_t* L_off, const int32_t* L_steps, const int32_t* L_cnt, int64_t n_L, int64_t K,
                                 const float* table, int64_t table_rows, const float* ff, const int64_t* F_pos, int64_t n_F,
                                 const float* sw, const int64_t* S_pos, int64_t n_S, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0 || n_hit < 0 || n_N < 0 || n_L < 0 || n_F < 0 || n_S < 0 || K < 0) return SRM2_ERR_ARG;
  if (n_hit + n_N + n_L + n_F + n_S == 0) return SRM2_OK;
  if (W == nullptr) return SRM2_ERR_ARG;
  if (n_hit > 0 && (pool == nullptr || hit_pos == nullptr || hit_slot == nullptr)) return SRM2_ERR_ARG;
  if (n_N > 0 && (fullN == nullptr || N_pos == nullptr || N_row == nullptr)) return SRM2_ERR_ARG;
  if (n_L > 0 && (fullL == nullptr || L_pos == nullptr || L_row == nullptr || L_off == nullptr || L_cnt == nullptr || table == nullptr ||
                  table_rows < 1 || (K > 0 && (logs == nullptr || L_steps == nullptr))))
    return SRM2_ERR_ARG;
  if (n_F > 0 && (ff == nullptr || F_pos == nullptr)) return SRM2_ERR_ARG;
  if (n_S > 0 && (sw == nullptr || S_pos == nullptr)) return SRM2_ERR_ARG;
  // the vector form only: callers fall back to the separate calls for other shapes
  if ((D & 3) != 0 || K > 8 || D > (1 << 20)) return SRM2_ERR_UNSUPPORTED;
  const void* al[] = {W, pool, fullN, fullL, logs, table, ff, sw};
  for (const void* p : al)
    if (p != nullptr && !aligned16(p)) return SRM2_ERR_UNSUPPORTED;
  AssembleArgs a{};
  a.W = W; a.D = (int)D; a.lpr = (int)(D / 4); a.shift = (a.lpr & (a.lpr - 1)) == 0 ? __builtin_ctz(a.lpr) : -1; a.K = (int)K;
  a.pool = pool; a.hit_pos = hit_pos; a.hit_slot = hit_slot;
  a.fullN = fullN; a.N_pos = N_pos; a.N_row = N_row; a.seed = seed; a.bound = bound;
  a.fullL = fullL; a.L_pos = L_pos; a.L_row = L_row; a.logs = logs; a.L_off = L_off; a.L_steps = L_steps; a.L_cnt = L_cnt;
  a.table = table; a.table_rows = table_rows; a.ff = ff; a.F_pos = F_pos; a.sw = sw; a.S_pos = S_pos; a.n = n;
  a.end_hit = n_hit * a.lpr; a.end_N = a.end_hit + n_N * a.lpr; a.end_L = a.end_N + n_L * a.lpr; a.end_F = a.end_L + n_F * a.lpr;
  a.end_S = a.end_F + n_S * a.lpr;
  const int64_t blocks = (a.end_S + 255) / 256;
  if (blocks > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K <= 4) srm2_assemble_kernel<4><<<(unsigned)blocks, 256, 0, st>>>(a);
  else srm2_assemble_kernel<8><<<(unsigned)blocks, 256, 0, st>>>(a);
  return launch_status();
}
