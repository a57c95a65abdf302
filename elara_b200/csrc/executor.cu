// The GPU half of the executor's update step as three kernels (srm2/elara.py:497-531 does it with ~25 index_select /
// index_put_ / index_copy_ / cat calls, three gpu_adam launches and as many temporaries):
//   hits    every resident row of the step: its gradient goes into the slot's resident history (when histories are
//           recorded) and through Adam into the pool — the gradient is read once, never materialised;
//   pack    everything that leaves the GPU, written straight into the three output buffers in the reference's order:
//             og  gradients of the S rows, then of the appended N rows, then of the appended L rows
//             of  updated full states of the compacted N and L rows and of the transient F rows (Adam applied on the
//                 way, same arithmetic as everywhere), then the full states of the evicted slots that go to M
//             oe  the valid resident-history entries of the evicted slots that go back to L
//           Evicted slots are read here, after the hits kernel (a row may be hit and evicted in the same step) and
//           before the admissions kernel (which reuses their slots and history rows);
//   admit   Adam on the admitted N / L / F rows written into their new pool slots, and the admission gradient as entry 0
//           of the new slot's resident history.
// One thread per 16-byte lane of one row; the groups are consecutive ranges of the item space.
#include "common.cuh"
#include "exact.cuh"

namespace srm2 {

struct UpdArgs {
  srm2_update u;
  int lpr, shift;
  int64_t rec;                              // 3 * D
  // pack: exclusive ends of the item ranges (in lanes): og | N cmp | L cmp | F not admitted | evicted to M | oe
  int64_t e_og, e_Nc, e_Lc, e_Fn, e_ev, e_oe;
  // admit: N adm | L adm | F adm
  int64_t e_Na, e_La, e_Fa;
};

__device__ __forceinline__ void split(const UpdArgs& a, int64_t t, int64_t& i, int& j) {
  if (a.shift >= 0) { i = t >> a.shift; j = (int)(t & (a.lpr - 1)) * 4; } else { i = t / a.lpr; j = (int)(t - i * a.lpr) * 4; }
}
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }

__global__ void __launch_bounds__(256) srm2_update_hits_kernel(UpdArgs a) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= a.u.n_hit * a.lpr) return;
  int64_t i; int j;
  split(a, t, i, j);
  const int64_t D = a.u.D;
  const float4 g = ld_stream4(a.u.G + a.u.hit_pos[i] * D + j);
  if (a.u.evl) st4(a.u.glog + (a.u.hrec_dyn[i] * a.u.K + a.u.hrec_j[i]) * D + j, g);
  float* b = a.u.pool + a.u.hit_slot[i] * a.rec + j;
  float4 w = ld4(b), m = ld4(b + D), v = ld4(b + 2 * D);
  const AdamSc sc{a.u.sc[0], a.u.sc[1], a.u.sc[2], a.u.sc[3], a.u.sc[4], a.u.sc[5], a.u.sc[6], a.u.sc[7]};
  adam_vec4_fast(w, m, v, g, adam_fast_prepare(sc));
  st4(b, w); st4(b + D, m); st4(b + 2 * D, v);
}

// Adam on record `src` with gradient row `g`, result to `dst` (a [3, D] record), this lane only.
__device__ __forceinline__ void adam_to(const UpdArgs& a, const float* src, const float* g, float* dst, int j) {
  const int64_t D = a.u.D;
  float4 w = ld_stream4(src + j), m = ld_stream4(src + D + j), v = ld_stream4(src + 2 * D + j);
  const AdamSc sc{a.u.sc[0], a.u.sc[1], a.u.sc[2], a.u.sc[3], a.u.sc[4], a.u.sc[5], a.u.sc[6], a.u.sc[7]};
  adam_vec4_fast(w, m, v, ld_stream4(g + j), adam_fast_prepare(sc));
  st4(dst + j, w); st4(dst + D + j, m); st4(dst + 2 * D + j, v);
}

__global__ void __launch_bounds__(256) srm2_update_pack_kernel(UpdArgs a) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= a.e_oe) return;
  const srm2_update& u = a.u;
  const int64_t D = u.D;
  int64_t i; int j;
  if (t < a.e_og) {                                      // og: S rows, appended N rows, appended L rows
    split(a, t, i, j);
    int64_t pos;
    if (i < u.n_S) pos = u.S_pos[i];
    else if (i < u.n_S + u.nNp) pos = u.N_pos[u.nNa + (i - u.n_S)];
    else pos = u.L_pos[u.nLa + (i - u.n_S - u.nNp)];
    st_stream4(u.og + i * D + j, ld_stream4(u.G + pos * D + j));
  } else if (t < a.e_Nc) {                               // compacted N rows
    split(a, t - a.e_og, i, j);
    const int64_t r = u.nNa + u.nNp + i;
    adam_to(a, u.fullN + r * a.rec, u.G + u.N_pos[r] * D, u.of + i * a.rec, j);
  } else if (t < a.e_Lc) {                               // compacted L rows
    split(a, t - a.e_Nc, i, j);
    const int64_t r = u.nLa + u.nLp + i;
    adam_to(a, u.fullL + r * a.rec, u.G + u.L_pos[r] * D, u.of + (u.nNc + i) * a.rec, j);
  } else if (t < a.e_Fn) {                               // transient F rows
    split(a, t - a.e_Lc, i, j);
    const int64_t r = u.nFa + i;
    adam_to(a, u.ff + r * a.rec, u.G + u.F_pos[r] * D, u.of + (u.nNc + u.nLc + i) * a.rec, j);
  } else if (t < a.e_ev) {                               // evicted slots that go to M: their full states
    split(a, t - a.e_Fn, i, j);
    const float* s = u.pool + u.evM_slot[i] * a.rec + j;
    float* d = u.of + (u.nNc + u.nLc + u.nFn + i) * a.rec + j;
    st_stream4(d, ld4(s)); st_stream4(d + D, ld4(s + D)); st_stream4(d + 2 * D, ld4(s + 2 * D));
  } else {                                               // evicted slots that go back to L: their valid history entries
    split(a, t - a.e_ev, i, j);
    st_stream4(u.oe + i * D + j, ld4(u.glog + u.evl_src[i] * D + j));
  }
}

__global__ void __launch_bounds__(256) srm2_update_admit_kernel(UpdArgs a) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= a.e_Fa) return;
  const srm2_update& u = a.u;
  const int64_t D = u.D;
  int64_t i; int j;
  if (t < a.e_Na) {
    split(a, t, i, j);
    const float* g = u.G + u.N_pos[i] * D;
    adam_to(a, u.fullN + i * a.rec, g, u.pool + u.N_adm_slot[i] * a.rec, j);
    if (u.evl) st4(u.glog + u.adm_rec_dyn[i] * u.K * D + j, ld_stream4(g + j));
  } else if (t < a.e_La) {
    split(a, t - a.e_Na, i, j);
    const float* g = u.G + u.L_pos[i] * D;
    adam_to(a, u.fullL + i * a.rec, g, u.pool + u.L_adm_slot[i] * a.rec, j);
    if (u.evl) st4(u.glog + u.adm_rec_dyn[u.nNa + i] * u.K * D + j, ld_stream4(g + j));
  } else {
    split(a, t - a.e_La, i, j);
    adam_to(a, u.ff + i * a.rec, u.G + u.F_pos[i] * D, u.pool + u.F_adm_slot[i] * a.rec, j);
  }
}

}  // namespace srm2

extern "C" int srm2_executor_update_f32(const srm2_update* up, srm2_stream_t stream) {
  using namespace srm2;
  if (up == nullptr) return SRM2_ERR_ARG;
  const srm2_update& u = *up;
  const int64_t counts[] = {u.n_hit, u.n_S, u.nNa, u.nNp, u.nNc, u.nLa, u.nLp, u.nLc, u.nFa, u.nFn, u.n_evM, u.n_evl};
  for (int64_t c : counts)
    if (c < 0) return SRM2_ERR_ARG;
  if (u.D <= 0 || u.K < 0) return SRM2_ERR_ARG;
  if ((u.D & 3) != 0 || u.D > (1 << 20)) return SRM2_ERR_UNSUPPORTED;
  const int64_t nN = u.nNa + u.nNp + u.nNc, nL = u.nLa + u.nLp + u.nLc, nF = u.nFa + u.nFn;
  const int64_t n_og = u.n_S + u.nNp + u.nLp, n_of = u.nNc + u.nLc + u.nFn + u.n_evM;
  const bool any = u.n_hit + nN + nL + nF + n_og + n_of + u.n_evl > 0;
  if (!any) return SRM2_OK;
  if (u.G == nullptr && (u.n_hit + nN + nL + nF + u.n_S > 0)) return SRM2_ERR_ARG;
  if ((u.n_hit > 0 || u.n_evM > 0 || u.nNa + u.nLa + u.nFa > 0) && u.pool == nullptr) return SRM2_ERR_ARG;
  if (u.n_hit > 0 && (u.hit_pos == nullptr || u.hit_slot == nullptr || (u.evl && (u.hrec_dyn == nullptr || u.hrec_j == nullptr)))) return SRM2_ERR_ARG;
  if ((u.evl && (u.n_hit > 0 || u.nNa + u.nLa > 0) || u.n_evl > 0) && u.glog == nullptr) return SRM2_ERR_ARG;
  if (nN > 0 && (u.fullN == nullptr || u.N_pos == nullptr)) return SRM2_ERR_ARG;
  if (nL > 0 && (u.fullL == nullptr || u.L_pos == nullptr)) return SRM2_ERR_ARG;
  if (nF > 0 && (u.ff == nullptr || u.F_pos == nullptr)) return SRM2_ERR_ARG;
  if (u.n_S > 0 && u.S_pos == nullptr) return SRM2_ERR_ARG;
  if ((u.nNa > 0 && u.N_adm_slot == nullptr) || (u.nLa > 0 && u.L_adm_slot == nullptr) || (u.nFa > 0 && u.F_adm_slot == nullptr)) return SRM2_ERR_ARG;
  if (u.evl && u.nNa + u.nLa > 0 && u.adm_rec_dyn == nullptr) return SRM2_ERR_ARG;
  if ((n_og > 0 && u.og == nullptr) || (n_of > 0 && u.of == nullptr) || (u.n_evl > 0 && (u.oe == nullptr || u.evl_src == nullptr))) return SRM2_ERR_ARG;
  if (u.n_evM > 0 && u.evM_slot == nullptr) return SRM2_ERR_ARG;
  const void* al[] = {u.G, u.pool, u.glog, u.fullN, u.fullL, u.ff, u.og, u.of, u.oe};
  for (const void* p : al)
    if (p != nullptr && !aligned16(p)) return SRM2_ERR_UNSUPPORTED;
  UpdArgs a{};
  a.u = u; a.lpr = (int)(u.D / 4); a.shift = (a.lpr & (a.lpr - 1)) == 0 ? __builtin_ctz(a.lpr) : -1; a.rec = 3 * u.D;
  const int64_t l = a.lpr;
  a.e_og = n_og * l; a.e_Nc = a.e_og + u.nNc * l; a.e_Lc = a.e_Nc + u.nLc * l; a.e_Fn = a.e_Lc + u.nFn * l;
  a.e_ev = a.e_Fn + u.n_evM * l; a.e_oe = a.e_ev + u.n_evl * l;
  a.e_Na = u.nNa * l; a.e_La = a.e_Na + u.nLa * l; a.e_Fa = a.e_La + u.nFa * l;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto blocks = [](int64_t items) { return (items + 255) / 256; };
  if (blocks(u.n_hit * l) > 0x7fffffffLL || blocks(a.e_oe) > 0x7fffffffLL || blocks(a.e_Fa) > 0x7fffffffLL) return SRM2_ERR_UNSUPPORTED;
  int launches = 0;
  if (u.n_hit > 0) { srm2_update_hits_kernel<<<(unsigned)blocks(u.n_hit * l), 256, 0, st>>>(a); ++launches; }
  if (a.e_oe > 0) { srm2_update_pack_kernel<<<(unsigned)blocks(a.e_oe), 256, 0, st>>>(a); ++launches; }
  if (a.e_Fa > 0) { srm2_update_admit_kernel<<<(unsigned)blocks(a.e_Fa), 256, 0, st>>>(a); ++launches; }
  return launch_status(launches);
}
