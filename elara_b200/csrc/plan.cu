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
