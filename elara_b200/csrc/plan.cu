// Classification and class partition of a step's unique rows: the part of ELARAPlanner.plan (srm2/elara.py:214-219,
// 229-239, 243, 258) that the reference runs as ~40 elementwise / searchsorted / where / bincount / argsort ops.
//   classify : one thread per unique row: pool slot and hit, membership in the look-ahead lists (binary search),
//              admission, directory code, table threshold, the 10-way class; class counts by warp-aggregated atomics
//   partition: order = stable argsort of the class = one 4-bit pass of the radix sort
// Integer work only: any correct implementation gives the reference's bits.
#include "common.cuh"
#include "scan.cuh"
#include "sort.cuh"

namespace srm2 {

constexpr int kMaxNext = 8;
struct NextLists { const int64_t* p[kMaxNext]; int64_t n[kMaxNext]; int count; };
enum : int { C_HIT = 0, C_NADM, C_NAPP, C_NCMP, C_LADM, C_LAPP, C_LCMP, C_FADM, C_FNADM, C_S };   // srm2/elara.py:32

// number of elements < v (side_right: <= v) in the ascending array a[0, n)
__device__ __forceinline__ int64_t bound(const int64_t* __restrict__ a, int64_t n, int64_t v, bool side_right) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    const int64_t x = __ldg(a + mid);
    if (side_right ? x <= v : x < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(256)
srm2_plan_classify_kernel(const int64_t* __restrict__ u, int64_t n, int64_t R, const int32_t* __restrict__ slot_of,
                          const int32_t* __restrict__ last_seen, const int8_t* __restrict__ code, const int8_t* __restrict__ kthr,
                          const int64_t* __restrict__ toff, int64_t T, NextLists nx, int64_t s, int K, int ttl, int want_T, int use_admit,
                          int32_t* __restrict__ sl_out, uint8_t* __restrict__ in_next_out, uint8_t* __restrict__ admit_io,
                          int8_t* __restrict__ c_out, int8_t* __restrict__ cls_out, int64_t* __restrict__ key_out,
                          unsigned long long* __restrict__ counts) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const bool live = i < n;
  int cls = 10;                                            // slot 10 counts row ids outside [0, R): nothing is read for them
  if (live) {
    const int64_t r = u[i];
    if (r >= 0 && r < R) {
      const int32_t sl = slot_of[r];
      const bool hit = sl >= 0;
      bool in_next = false;
      for (int q = 0; q < nx.count; ++q) {
        if (nx.n[q] <= 0) continue;
        int64_t j = bound(nx.p[q], nx.n[q], r, false);
        if (j > nx.n[q] - 1) j = nx.n[q] - 1;
        in_next |= __ldg(nx.p[q] + j) == r;
      }
      const bool admit = use_admit ? admit_io[i] != 0 : (!hit && (ttl ? (int64_t)last_seen[r] > s : in_next));
      const int c = code[r];
      int64_t t = bound(toff, T, r, true) - 1;
      if (t < 0) t += T;                                   // the reference's negative index wraps (never happens with toff[0] = 0)
      const int thr = kthr[t];
      const bool isN = c == 0, isL = c >= 1 && c <= K, app = c < thr;
      cls = C_S;
      if (!isN && !isL && (admit || want_T)) cls = admit ? C_FADM : C_FNADM;
      if (isL) cls = admit ? C_LADM : (app ? C_LAPP : C_LCMP);
      if (isN) cls = admit ? C_NADM : (app ? C_NAPP : C_NCMP);
      if (hit) cls = C_HIT;
      sl_out[i] = sl; in_next_out[i] = in_next; admit_io[i] = admit; c_out[i] = (int8_t)c;
    } else {
      sl_out[i] = -1; in_next_out[i] = 0; admit_io[i] = 0; c_out[i] = 0;
    }
    cls_out[i] = (int8_t)(cls < 10 ? cls : C_S);
    key_out[i] = cls < 10 ? cls : C_S;
  }
  const unsigned act = __ballot_sync(0xffffffffu, live);
  if (live) {
    const unsigned m = __match_any_sync(act, cls);
    if ((threadIdx.x & 31) == __ffs(m) - 1) atomicAdd(counts + cls, (unsigned long long)__popc(m));
  }
}

__global__ void __launch_bounds__(256)
srm2_plan_order_kernel(const uint32_t* __restrict__ spos, int64_t n, int64_t* __restrict__ order) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n) order[i] = spos[i];
}

constexpr int kPlanBits = 4;
static size_t plan_align(size_t x) { return (x + 255) / 256 * 256; }
static size_t plan_layout(int64_t n, char* base, SortBuffers* sb, int64_t** key64) {
  const int tiles = sort_tiles(n > 0 ? n : 1);
  const size_t nn = (size_t)(n > 0 ? n : 1);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = plan_align(off + bytes); return o; };
  const size_t o_k = take(nn * 8), o_ka = take(nn * 4), o_va = take(nn * 4), o_h = take(sort_hist_words(tiles, kPlanBits) * 4),
               o_dt = take(sort_dtot_words(tiles, kPlanBits, 1) * 4);
  if (sb) {
    auto w = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    sb->keyA = w(o_ka); sb->valA = w(o_va); sb->keyB = nullptr; sb->valB = nullptr; sb->hist = w(o_h); sb->dtot = w(o_dt); sb->tiles = tiles;
    *key64 = reinterpret_cast<int64_t*>(base + o_k);
  }
  return off;
}

// ---- eviction candidates (srm2/elara.py:220-228, 245-246) --------------------------------------------------------------
// protect = pinned | (slots named by the look-ahead lists); a dynamic slot expires when it is not protected (TTL mode: and
// its row was last seen at or before step s); the dynamic slots are then split, in order, into expired | kept.
__global__ void __launch_bounds__(256)
srm2_plan_protect_kernel(NextLists nx, int64_t total, const int32_t* __restrict__ slot_of, int64_t R, uint8_t* __restrict__ protect, int64_t C) {
  int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= total) return;
  int q = 0;
  while (q < nx.count - 1 && t >= nx.n[q]) { t -= nx.n[q]; ++q; }
  const int64_t r = nx.p[q][t];
  if (r < 0 || r >= R) return;
  const int32_t sn = slot_of[r];
  if (sn >= 0 && sn < C) protect[sn] = 1;                 // every writer stores the same value
}

__global__ void __launch_bounds__(256)
srm2_plan_expired_kernel(const int64_t* __restrict__ dyn_slots, int64_t nd, const uint8_t* __restrict__ protect, int64_t C,
                         const int64_t* __restrict__ slot_row, const int32_t* __restrict__ last_seen, int64_t R, int64_t s, int ttl,
                         uint8_t* __restrict__ exp_out, int64_t* __restrict__ key_out) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= nd) return;
  const int64_t sl = dyn_slots[i];
  bool e = false;
  if (sl >= 0 && sl < C) {
    e = protect[sl] == 0;
    if (ttl) {
      int64_t row = slot_row[sl];
      if (row < 0) row += R;                               // the reference's negative index wraps
      e = e && row >= 0 && row < R && (int64_t)last_seen[row] <= s;
    }
  }
  exp_out[i] = e; key_out[i] = e ? 0 : 1;                  // expired slots first, order kept inside both groups
}

// parted[i] = dyn_slots[order[i]]; n_exp = number of keys 0 (digit total, or the scanned start of digit 1)
__global__ void __launch_bounds__(256)
srm2_plan_split_kernel(const int64_t* __restrict__ dyn_slots, const uint32_t* __restrict__ spos, int64_t nd, const uint32_t* __restrict__ dtot,
                       const uint32_t* __restrict__ hist, int tiles, int64_t* __restrict__ parted, int64_t* __restrict__ n_exp) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i == 0) *n_exp = dtot ? (int64_t)dtot[0] : (int64_t)hist[tiles];
  if (i < nd) parted[i] = dyn_slots[spos[i]];
}

// ---- packed eviction outputs and host work lists (srm2/elara.py:389-407) ------------------------------------------------
// Two stable one-bit partitions (evicted rows going to M first; valid resident-history entries first) and one kernel
// that writes every list of the plan's single device-to-host copy into one flat buffer.
struct PackArgs {
  const int64_t* ev_slot; const uint8_t* rep; const int64_t* evf_slots; const int64_t* evl_ids; const int64_t* ev_dyn; int64_t nev; int K;
  const int32_t* loc; int64_t n_loc; const int64_t* F_row; int64_t nF; int64_t nFa; const int64_t* S_row; int64_t nS;
  const int64_t* c_slots; int64_t nc; const int32_t* L_ids; int64_t nLK; const int64_t* a_ids; int64_t na;
  const int64_t* mat_top; const int64_t* log_top; const int64_t* live;
  const uint32_t* om; const uint32_t* ol; const unsigned long long* rep_sum;
  int64_t* evM_slot; int64_t* evl_src; int64_t* flat;
  int64_t end[9];                                   // exclusive ends of the item ranges: the 7 flat parts, evM_slot, evl_src
};

__global__ void __launch_bounds__(256)
srm2_plan_pack_keys_kernel(const uint8_t* __restrict__ rep, int64_t nev, const int64_t* __restrict__ evl_ids, int64_t nevK,
                           int64_t* __restrict__ key1, int64_t* __restrict__ key2, unsigned long long* __restrict__ rep_sum) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  const bool r = i < nev && rep[i] != 0;
  if (i < nev) key1[i] = r ? 1 : 0;
  if (i < nevK) key2[i] = evl_ids[i] < 0 ? 1 : 0;
  const unsigned m = __ballot_sync(0xffffffffu, r);
  if ((threadIdx.x & 31) == 0 && m) atomicAdd(rep_sum, (unsigned long long)__popc(m));
}

__device__ __forceinline__ int64_t loc_of(const PackArgs& a, int64_t row) {
  if (row < 0) row += a.n_loc;                            // the reference's negative index wraps
  return (row >= 0 && row < a.n_loc) ? (int64_t)a.loc[row] : -1;
}

__global__ void __launch_bounds__(256)
srm2_plan_pack_kernel(PackArgs a) {
  const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (t >= a.end[8]) return;
  if (t < a.end[0]) { a.flat[t] = loc_of(a, a.S_row[t]); return; }
  if (t < a.end[1]) { a.flat[t] = loc_of(a, a.F_row[t - a.end[0]]); return; }
  if (t < a.end[2]) { a.flat[t] = (int64_t)a.L_ids[t - a.end[1]]; return; }
  if (t < a.end[3]) { a.flat[t] = a.a_ids[t - a.end[2]]; return; }
  if (t < a.end[4]) {                                      // W_slot: compactions, transient M updates, evictions
    const int64_t i = t - a.end[3], nFn = a.nF - a.nFa;
    int64_t v;
    if (i < a.nc) v = a.c_slots[i];
    else if (i < a.nc + nFn) v = loc_of(a, a.F_row[a.nFa + (i - a.nc)]);
    else v = a.evf_slots[a.om[i - a.nc - nFn]];
    a.flat[t] = v; return;
  }
  if (t < a.end[5]) { a.flat[t] = a.evl_ids[a.ol[t - a.end[4]]]; return; }
  if (t < a.end[6]) {
    const int q = (int)(t - a.end[5]);
    a.flat[t] = q == 0 ? *a.mat_top : q == 1 ? *a.log_top : q == 2 ? *a.live : (int64_t)*a.rep_sum;
    return;
  }
  if (t < a.end[7]) { const int64_t i = t - a.end[6]; a.evM_slot[i] = a.ev_slot[a.om[i]]; return; }
  const int64_t j = t - a.end[7];
  const uint32_t o = a.ol[j];
  a.evl_src[j] = a.ev_dyn[o / (uint32_t)a.K] * a.K + (o % (uint32_t)a.K);
}

static size_t pack_layout(int64_t nev, int64_t K, size_t* o2, size_t* oc) {
  const size_t l1 = plan_layout(nev, nullptr, nullptr, nullptr), l2 = plan_layout(nev * K, nullptr, nullptr, nullptr);
  if (o2) *o2 = l1;
  if (oc) *oc = l1 + l2;
  return l1 + l2 + 256;
}

}  // namespace srm2

extern "C" size_t srm2_plan_scratch_bytes(int64_t n) { return n < 0 ? 0 : srm2::plan_layout(n, nullptr, nullptr, nullptr); }

extern "C" int srm2_plan_classify(const int64_t* u, int64_t n, int64_t R, const int32_t* slot_of, const int32_t* last_seen, const int8_t* code,
                                  const int8_t* kthr, const int64_t* toff, int64_t T, const int64_t* const* u_next, const int64_t* n_next,
                                  int64_t n_lists, int64_t s, int64_t K, int ttl, int want_T, int use_admit, int32_t* sl, uint8_t* in_next,
                                  uint8_t* admit, int8_t* c, int8_t* cls, int64_t* counts, int64_t* order, void* scratch,
                                  size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || R < 0 || T < 1 || n_lists < 0 || n_lists > kMaxNext || counts == nullptr || (n_lists > 0 && (u_next == nullptr || n_next == nullptr)))
    return SRM2_ERR_ARG;
  if (n > 0 && (u == nullptr || slot_of == nullptr || code == nullptr || kthr == nullptr || toff == nullptr || sl == nullptr || in_next == nullptr ||
                admit == nullptr || c == nullptr || cls == nullptr || order == nullptr || (ttl && !use_admit && last_seen == nullptr)))
    return SRM2_ERR_ARG;
  if (n >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < plan_layout(n, nullptr, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (note_cuda(cudaMemsetAsync(counts, 0, 11 * 8, st))) return SRM2_ERR_CUDA;
  if (n == 0) return SRM2_OK;
  NextLists nx{};
  nx.count = (int)n_lists;
  for (int q = 0; q < nx.count; ++q) {
    if (n_next[q] < 0 || (n_next[q] > 0 && u_next[q] == nullptr)) return SRM2_ERR_ARG;
    nx.p[q] = u_next[q]; nx.n[q] = n_next[q];
  }
  SortBuffers sb; int64_t* key64 = nullptr;
  plan_layout(n, static_cast<char*>(scratch), &sb, &key64);
  if (note_cuda(cudaMemsetAsync(sb.dtot, 0, sort_dtot_words(sb.tiles, kPlanBits, 1) * 4, st))) return SRM2_ERR_CUDA;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  srm2_plan_classify_kernel<<<blocks, 256, 0, st>>>(u, n, R, slot_of, last_seen, code, kthr, toff, T, nx, s, (int)K, ttl, want_T, use_admit, sl, in_next,
                                                    admit, c, cls, key64, reinterpret_cast<unsigned long long*>(counts));
  int launches = 1;
  const uint32_t *skey = nullptr, *spos = nullptr, *dt = nullptr;
  const int rc = radix_sort_by_key(key64, n, nullptr, 0, 16, kPlanBits, 1, sb, &skey, &spos, &dt, &launches, st);
  if (rc != SRM2_OK) return rc;
  srm2_plan_order_kernel<<<blocks, 256, 0, st>>>(spos, n, order);
  return launch_status(launches + 1);
}

extern "C" int srm2_plan_evict_candidates(const int64_t* const* u_next, const int64_t* n_next, int64_t n_lists, const int32_t* slot_of, int64_t R,
                                          const uint8_t* pinned, int64_t C, const int64_t* dyn_slots, int64_t nd, const int64_t* slot_row,
                                          const int32_t* last_seen, int64_t s, int ttl, uint8_t* protect, uint8_t* exp, int64_t* n_exp,
                                          int64_t* parted, void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (n_lists < 0 || n_lists > kMaxNext || R < 0 || C < 0 || nd < 0 || n_exp == nullptr || (n_lists > 0 && (u_next == nullptr || n_next == nullptr)))
    return SRM2_ERR_ARG;
  if (C > 0 && (pinned == nullptr || protect == nullptr)) return SRM2_ERR_ARG;
  if (nd > 0 && (dyn_slots == nullptr || slot_row == nullptr || exp == nullptr || parted == nullptr || (ttl && last_seen == nullptr))) return SRM2_ERR_ARG;
  if (nd >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < plan_layout(nd, nullptr, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  NextLists nx{};
  int64_t total = 0;
  for (int q = 0; q < (int)n_lists; ++q) {
    if (n_next[q] < 0 || (n_next[q] > 0 && (u_next[q] == nullptr || slot_of == nullptr))) return SRM2_ERR_ARG;
    if (n_next[q] == 0) continue;
    nx.p[nx.count] = u_next[q]; nx.n[nx.count] = n_next[q]; ++nx.count; total += n_next[q];
  }
  int launches = 0;
  if (C > 0 && note_cuda(cudaMemcpyAsync(protect, pinned, (size_t)C, cudaMemcpyDeviceToDevice, st))) return SRM2_ERR_CUDA;
  if (total > 0 && C > 0) {
    srm2_plan_protect_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(nx, total, slot_of, R, protect, C);
    ++launches;
  }
  if (nd == 0) {
    if (note_cuda(cudaMemsetAsync(n_exp, 0, 8, st))) return SRM2_ERR_CUDA;
    return launch_status(launches);
  }
  SortBuffers sb; int64_t* key64 = nullptr;
  plan_layout(nd, static_cast<char*>(scratch), &sb, &key64);
  if (note_cuda(cudaMemsetAsync(sb.dtot, 0, sort_dtot_words(sb.tiles, kPlanBits, 1) * 4, st))) return SRM2_ERR_CUDA;
  const unsigned blocks = (unsigned)((nd + 255) / 256);
  srm2_plan_expired_kernel<<<blocks, 256, 0, st>>>(dyn_slots, nd, protect, C, slot_row, last_seen, R, s, ttl, exp, key64);
  const uint32_t *skey = nullptr, *spos = nullptr, *dt = nullptr;
  const int rc = radix_sort_by_key(key64, nd, nullptr, 0, 2, 1, 1, sb, &skey, &spos, &dt, &launches, st);
  if (rc != SRM2_OK) return rc;
  srm2_plan_split_kernel<<<blocks, 256, 0, st>>>(dyn_slots, spos, nd, dt, sb.hist, sb.tiles, parted, n_exp);
  return launch_status(launches + 2);
}

extern "C" size_t srm2_plan_pack_scratch_bytes(int64_t nev, int64_t K) {
  return (nev < 0 || K < 1) ? 0 : srm2::pack_layout(nev, K, nullptr, nullptr);
}

extern "C" int srm2_plan_pack(const int64_t* ev_slot, const uint8_t* rep, const int64_t* evf_slots, const int64_t* evl_ids, const int64_t* ev_dyn,
                              int64_t nev, int64_t K, const int32_t* loc, int64_t n_loc, const int64_t* F_row, int64_t nF, int64_t nFa,
                              const int64_t* S_row, int64_t nS, const int64_t* c_slots, int64_t nc, const int32_t* L_ids, int64_t nL,
                              const int64_t* a_ids, int64_t na, const int64_t* mat_top, const int64_t* log_top, const int64_t* live,
                              int64_t* evM_slot, int64_t* evl_src, int64_t* flat, void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (nev < 0 || K < 1 || K > 64 || n_loc < 0 || nF < 0 || nFa < 0 || nFa > nF || nS < 0 || nc < 0 || nL < 0 || na < 0 || flat == nullptr ||
      mat_top == nullptr || log_top == nullptr || live == nullptr)
    return SRM2_ERR_ARG;
  if (nev > 0 && (ev_slot == nullptr || rep == nullptr || evf_slots == nullptr || evl_ids == nullptr || ev_dyn == nullptr || evM_slot == nullptr ||
                  evl_src == nullptr))
    return SRM2_ERR_ARG;
  if ((nF > 0 && (F_row == nullptr || loc == nullptr)) || (nS > 0 && (S_row == nullptr || loc == nullptr)) || (nc > 0 && c_slots == nullptr) ||
      (nL > 0 && L_ids == nullptr) || (na > 0 && a_ids == nullptr))
    return SRM2_ERR_ARG;
  if (nev * K >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  size_t o2 = 0, oc = 0;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < pack_layout(nev, K, &o2, &oc)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(scratch);
  unsigned long long* rep_sum = reinterpret_cast<unsigned long long*>(base + oc);
  if (note_cuda(cudaMemsetAsync(rep_sum, 0, 8, st))) return SRM2_ERR_CUDA;
  int launches = 0;
  const uint32_t *om = nullptr, *ol = nullptr;
  if (nev > 0) {
    SortBuffers sb1, sb2; int64_t *key1 = nullptr, *key2 = nullptr;
    plan_layout(nev, base, &sb1, &key1);
    plan_layout(nev * K, base + o2, &sb2, &key2);
    if (note_cuda(cudaMemsetAsync(sb1.dtot, 0, sort_dtot_words(sb1.tiles, kPlanBits, 1) * 4, st))) return SRM2_ERR_CUDA;
    if (note_cuda(cudaMemsetAsync(sb2.dtot, 0, sort_dtot_words(sb2.tiles, kPlanBits, 1) * 4, st))) return SRM2_ERR_CUDA;
    srm2_plan_pack_keys_kernel<<<(unsigned)((nev * K + 255) / 256), 256, 0, st>>>(rep, nev, evl_ids, nev * K, key1, key2, rep_sum);
    ++launches;
    const uint32_t *sk = nullptr, *dt = nullptr;
    int rc = radix_sort_by_key(key1, nev, nullptr, 0, 2, 1, 1, sb1, &sk, &om, &dt, &launches, st);
    if (rc != SRM2_OK) return rc;
    rc = radix_sort_by_key(key2, nev * K, nullptr, 0, 2, 1, 1, sb2, &sk, &ol, &dt, &launches, st);
    if (rc != SRM2_OK) return rc;
  }
  PackArgs a{};
  a.ev_slot = ev_slot; a.rep = rep; a.evf_slots = evf_slots; a.evl_ids = evl_ids; a.ev_dyn = ev_dyn; a.nev = nev; a.K = (int)K;
  a.loc = loc; a.n_loc = n_loc; a.F_row = F_row; a.nF = nF; a.nFa = nFa; a.S_row = S_row; a.nS = nS; a.c_slots = c_slots; a.nc = nc;
  a.L_ids = L_ids; a.nLK = nL * K; a.a_ids = a_ids; a.na = na; a.mat_top = mat_top; a.log_top = log_top; a.live = live;
  a.om = om; a.ol = ol; a.rep_sum = rep_sum; a.evM_slot = evM_slot; a.evl_src = evl_src; a.flat = flat;
  const int64_t sizes[9] = {nS, nF, nL * K, na, nc + (nF - nFa) + nev, nev * K, 4, nev, nev * K};
  int64_t e = 0;
  for (int q = 0; q < 9; ++q) { e += sizes[q]; a.end[q] = e; }
  srm2_plan_pack_kernel<<<(unsigned)((e + 255) / 256), 256, 0, st>>>(a);
  return launch_status(launches + 1);
}
