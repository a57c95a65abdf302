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
