// Deterministic segment-reduce of per-lookup gradients into unique rows, in the summation order of
// PyTorch's CUDA aten::embedding_dense_backward (the operator the reference calls at srm2/train.py:429),
// optionally fused with the row-sparse Adam update of the rows (no [n_unique, D] gradient round trip).
//
// Order being reproduced (established by black-box runs of that operator on a B200, torch 2.11.0):
//   n  > 3072 lookups: the lookups of a unique row, in ascending lookup position, are cut into runs of 10; each run
//                      is summed left to right starting from +0; the run sums are added left to right from +0.
//   n <= 3072 lookups: lookups are walked in windows of 32 consecutive positions; inside a window the lookups of a row
//                      are summed left to right starting from the first; window sums are added to a row that starts +0.
//
// Pipeline (all on the caller's stream, nothing synchronises, scratch supplied by the caller):
//   1. stable LSD radix sort of (key = inverse index, value = lookup position); the number of passes follows from the
//      bound on the number of unique rows (two 9-bit passes for ~200 k lookups).
//   2. segment boundaries from the sorted keys.
//   3. plan: runs per segment and three block-local exclusive scans (runs, runs of multi-run rows, multi-run rows);
//      the last CTA to finish scans the per-CTA totals.  A global prefix is (CTA prefix + in-CTA offset): no separate
//      scan launch.
//   4. run descriptors {first sorted index, row, length, partial slot} and the list of multi-run rows.
//   5. run sums: one thread group per run sums its <= 10 gradient rows, all loads issued up front.  Work is spread over
//      the whole GPU however long the longest segment is.  Rows with one run are finished here (written, or Adam applied).
//   6. multi-run rows: the run sums are staged through shared memory with cp.async (a warp per short row, the whole CTA
//      per long row) and added in order; the only serial part is the fp32 add chain itself.
// Gradient rows are read exactly once (D*4 bytes per lookup); everything else is small integer traffic.
#include "common.cuh"
#include "exact.cuh"
#include "scan.cuh"
#include "sort.cuh"

namespace srm2 {

constexpr int kRun = 10;            // lookups per run (large inputs)
constexpr int kSmallN = 3072;       // inputs up to this many lookups use the windowed order
constexpr int kWindow = 32;
constexpr int kPlanThreads = 256;

struct SegCounters { uint32_t n_runs, n_mrows, n_mruns, done; };
constexpr int kMaxGradPeers = 16;
constexpr int kPeerShift = 24;      // pull mode: a lookup is named by (source rank << 24) | row in that rank's gradient buffer

struct ReduceArgs {
  const float* grad; int D; int lpr; int shift;
  const uint32_t* skey; const uint32_t* spos; const uint32_t* seg_start; const uint32_t* seg_end;
  const uint4* run_desc; const uint32_t* run_pos; const uint32_t* mrows; uint4* mrow_info; const SegCounters* counters; int inplace;
  const uint32_t* mrun_off; const uint32_t* bpre_m;
  float* partial;
  float* out;                                     // [nu, D] (unfused) or nullptr
  float* pool; const int64_t* slots; AdamSc sc;   // fused Adam: pool [C,3,D], slots[j] = pool row of unique row j
  int64_t nu_host; const int64_t* nu_dev; int64_t cap; int64_t n;
  const float* peer[kMaxGradPeers];               // pull mode: gradient buffers of all ranks (peer pointers), see grad_row
};

__device__ __forceinline__ int64_t load_nu(int64_t nu_host, const int64_t* nu_dev, int64_t cap) {
  int64_t nu = nu_dev ? *nu_dev : nu_host;
  return nu > cap ? cap : (nu < 0 ? 0 : nu);
}

__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// Address of a lookup's gradient row.  Local mode: `code` is the row of a.grad.  Pull mode: the row lives in the buffer
// of the rank that produced it and is read from there (peer memory over NVLink, plain 16-byte asynchronous copies).
template <bool PEER>
__device__ __forceinline__ const float* grad_row(const ReduceArgs& a, uint32_t code) {
  if (PEER) return a.peer[code >> kPeerShift] + (int64_t)(code & ((1u << kPeerShift) - 1u)) * a.D;
  return a.grad + (int64_t)code * a.D;
}

// Writes the finished gradient sum of unique row j (lane j4): either into out, or through Adam into the pool.
template <bool FUSED>
__device__ __forceinline__ void finish_row(const ReduceArgs& a, uint32_t j, int j4, const float4& g) {
  if (FUSED) {
    float* b = a.pool + a.slots[j] * (3 * (int64_t)a.D) + j4 * 4;
    float4 w = *reinterpret_cast<const float4*>(b), m = *reinterpret_cast<const float4*>(b + a.D),
           v = *reinterpret_cast<const float4*>(b + 2 * a.D);
    { const AdamSc sc = a.sc; adam_vec4_fast(w, m, v, g, adam_fast_prepare(sc)); }
    *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
  } else {
    *reinterpret_cast<float4*>(a.out + (int64_t)j * a.D + j4 * 4) = g;
  }
}

// ------------------------------------------------------------------------------------------ boundaries
// seg_start[j] / seg_end[j] = sorted index range of unique row j.  Both arrays are zeroed first, so a row that no
// lookup names has an empty range.  Lookups with an invalid index carry key == cap and belong to no row.
__global__ void __launch_bounds__(256)
srm2_segment_bounds_kernel(const uint32_t* __restrict__ skey, int64_t n_host, const int64_t* __restrict__ n_dev,
                           uint32_t* __restrict__ seg_start, uint32_t* __restrict__ seg_end, int64_t cap) {
  const int64_t n = eff_count(n_host, n_dev);
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const uint32_t k = skey[i];
  if ((int64_t)k >= cap) return;
  if (i == 0 || skey[i - 1] != k) seg_start[k] = (uint32_t)i;
  if (i == n - 1 || skey[i + 1] != k) seg_end[k] = (uint32_t)(i + 1);
}

// ------------------------------------------------------------------------------------------ plan
// Per unique row: runs, block-local exclusive offsets of (runs, runs of multi-run rows, multi-run rows); per CTA the
// totals; the last CTA to finish turns the totals into exclusive prefixes and writes the grand totals.
// Rows without lookups are finished here (zero gradient).
template <bool FUSED>
__global__ void __launch_bounds__(kPlanThreads)
srm2_segment_plan_kernel(ReduceArgs a, uint32_t* __restrict__ run_off, uint32_t* __restrict__ mrun_off,
                         uint32_t* __restrict__ mrow_off, uint32_t* __restrict__ bsum_r, uint32_t* __restrict__ bsum_m,
                         uint32_t* __restrict__ bsum_f, SegCounters* __restrict__ counters, int nblocks, int skip_empty) {
  __shared__ uint64_t ws[33];
  __shared__ bool last;
  const int64_t nu = load_nu(a.nu_host, a.nu_dev, a.cap);
  const int64_t j = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x;
  uint32_t r = 0, m = 0, f = 0;
  if (j < nu) {
    const uint32_t len = a.seg_end[j] - a.seg_start[j];
    r = (len + kRun - 1) / kRun; f = r > 1; m = f ? r : 0u;
    if (len == 0 && !skip_empty)
      for (int j4 = 0; j4 < a.lpr; ++j4) finish_row<FUSED>(a, (uint32_t)j, j4, make_float4(0.f, 0.f, 0.f, 0.f));
  }
  // the three counters scan as one packed word: runs | runs of multi-run rows | multi-run rows (21 bits each; the host
  // side rejects inputs whose totals would not fit)
  uint64_t tot;
  const uint64_t ex = block_exclusive_scan64<kPlanThreads>(((uint64_t)r << 42) | ((uint64_t)m << 21) | f, ws, &tot);
  constexpr uint64_t kM = (1ull << 21) - 1;
  if (j < a.cap) { run_off[j] = (uint32_t)(ex >> 42); mrun_off[j] = (uint32_t)((ex >> 21) & kM); mrow_off[j] = (uint32_t)(ex & kM); }
  if (threadIdx.x == 0) {
    bsum_r[blockIdx.x] = (uint32_t)(tot >> 42); bsum_m[blockIdx.x] = (uint32_t)((tot >> 21) & kM); bsum_f[blockIdx.x] = (uint32_t)(tot & kM);
    __threadfence();
    last = atomicAdd(&counters->done, 1u) == (uint32_t)(nblocks - 1);
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // per-CTA totals -> exclusive prefixes; these totals can exceed 21 bits, so they scan as three 64-bit sums
  uint64_t cr = 0, cm = 0, cf = 0;
  for (int base = 0; base < nblocks; base += kPlanThreads) {
    const int i = base + threadIdx.x;
    const uint64_t vr = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bsum_r)[i] : 0u;
    const uint64_t vm = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bsum_m)[i] : 0u;
    const uint64_t vf = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bsum_f)[i] : 0u;
    uint64_t t0, t1, t2;
    const uint64_t xr = block_exclusive_scan64<kPlanThreads>(vr, ws, &t0);
    const uint64_t xm = block_exclusive_scan64<kPlanThreads>(vm, ws, &t1);
    const uint64_t xf = block_exclusive_scan64<kPlanThreads>(vf, ws, &t2);
    if (i < nblocks) { bsum_r[i] = (uint32_t)(cr + xr); bsum_m[i] = (uint32_t)(cm + xm); bsum_f[i] = (uint32_t)(cf + xf); }
    cr += t0; cm += t1; cf += t2;
  }
  if (threadIdx.x == 0) { counters->n_runs = (uint32_t)cr; counters->n_mruns = (uint32_t)cm; counters->n_mrows = (uint32_t)cf; counters->done = 0u; }
}

// Run descriptors and the multi-run rows; one thread per sorted lookup, the first lookup of a run writes.
//   run_desc[c] = {x, length | kMultiBit, z, w};  x = the lookup position itself when the run has one lookup
//     run of a multi-run row: c = its partial slot (these runs come first), z = partial slot, w = index of the row in
//                             mrow_info;  single-run row: c = n_mruns + rank among single-run rows, (z, w) = 64-bit
//                             target: the pool row (fused) or the unique row index.
//   mrow_info[mi] = {unique row, number of runs, first partial slot, finished-run counter = 0}
constexpr uint32_t kMultiBit = 0x80000000u;
__global__ void __launch_bounds__(256)
srm2_segment_descr_kernel(const uint32_t* __restrict__ skey, const uint32_t* __restrict__ spos, int64_t n_host,
                          const int64_t* __restrict__ n_dev, const uint32_t* __restrict__ seg_start,
                          const uint32_t* __restrict__ seg_end, const uint32_t* __restrict__ run_off,
                          const uint32_t* __restrict__ mrun_off, const uint32_t* __restrict__ mrow_off,
                          const uint32_t* __restrict__ bpre_r, const uint32_t* __restrict__ bpre_m,
                          const uint32_t* __restrict__ bpre_f, const SegCounters* __restrict__ counters,
                          const int64_t* __restrict__ slots, const uint32_t* __restrict__ src_code,
                          uint4* __restrict__ run_desc, uint32_t* __restrict__ run_pos,
                          uint32_t* __restrict__ mrows, uint4* __restrict__ mrow_info, int64_t nu_host,
                          const int64_t* __restrict__ nu_dev, int64_t cap) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= eff_count(n_host, n_dev)) return;
  const uint32_t j = skey[i];
  if ((int64_t)j >= load_nu(nu_host, nu_dev, cap)) return;
  const uint32_t s = seg_start[j], e = seg_end[j];
  const uint32_t off = (uint32_t)i - s;
  const bool multi = e - s > (uint32_t)kRun;
  const uint32_t blk = j / kPlanThreads, ri = off / kRun, rq = off - ri * kRun;
  const uint32_t rbase = bpre_r[blk] + run_off[j], mbase = bpre_m[blk] + mrun_off[j];
  const uint32_t c = multi ? mbase + ri : counters->n_mruns + (rbase - mbase);
  // what names the lookup's gradient row from here on: its position, or in pull mode its (rank, row) code
  const uint32_t code = src_code ? src_code[spos[i]] : spos[i];
  run_pos[(int64_t)c * kRun + rq] = code;                // rows of run c, padded to kRun per run
  if (rq != 0) return;
  const uint32_t len = min((uint32_t)kRun, e - (uint32_t)i);
  if (multi) {
    const uint32_t mi = bpre_f[blk] + mrow_off[j];
    run_desc[c] = make_uint4(len == 1 ? code : (uint32_t)i, len | kMultiBit, c, mi);
    if (off == 0) { mrows[mi] = j; mrow_info[mi] = make_uint4(j, (e - s + kRun - 1) / kRun, mbase, 0u); }
  } else {
    const uint64_t target = slots ? (uint64_t)slots[j] : (uint64_t)j;
    run_desc[c] = make_uint4(len == 1 ? code : (uint32_t)i, len, (uint32_t)target, (uint32_t)(target >> 32));
  }
}

// ------------------------------------------------------------------------------------------ run sums
// Finishes a row whose state (fused) was loaded ahead of time.
template <bool FUSED>
__device__ __forceinline__ void finish_loaded(const ReduceArgs& a, float* b, float4 w, float4 m, float4 v, const float4& g) {
  if (FUSED) {
    { const AdamSc sc = a.sc; adam_vec4_fast(w, m, v, g, adam_fast_prepare(sc)); }
    *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
  } else {
    *reinterpret_cast<float4*>(b) = g;
  }
}

// One thread per (run, 16-byte lane).  Sums the <= 10 gradient rows of the run from +0.
//  - single-run row: finished here ((+0) + run sum); its (w, m, v) loads are issued together with the gradient loads;
//  - run of a multi-run row: the run sum goes to the partial buffer.  With a.inplace (the D/4 lanes of a run are an
//    aligned part of one warp) the group then counts itself finished on the row; the group that completes the row adds
//    the row's run sums in order and finishes the row — nobody waits, and the long rows (whose runs come first in the
//    descriptor order) are finished while the bulk of the single-run rows is still streaming.  Without a.inplace a
//    separate kernel adds the run sums.
struct RunItem { uint4 d; uint2 p[kRun / 2]; };

__device__ __forceinline__ void load_item(const ReduceArgs& a, int64_t c, RunItem& it) {
  it.d = __ldg(a.run_desc + c);
  const uint2* pp = reinterpret_cast<const uint2*>(a.run_pos + c * kRun);
#pragma unroll
  for (int q = 0; q < kRun / 2; ++q) it.p[q] = __ldg(pp + q);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

#ifndef SRM2_RUN_PREFETCH
#define SRM2_RUN_PREFETCH 1
#endif
constexpr bool kRunPrefetch = SRM2_RUN_PREFETCH != 0;
constexpr int kInplaceMaxRuns = 512;      // rows with more runs (> 5120 lookups) are finished by a whole CTA after its last item
                                          // instead of the lane group that completed them: 256 threads copy ten times more
                                          // at once; shorter chains hide behind the single-run rows still streaming
constexpr int kRunThreads = 256;
constexpr int kRunStageVecs = kRun + 3;                                  // gradient rows + w, m, v
constexpr int kLongCap = 16;              // long rows one CTA can take over; further ones are finished by their lane group
constexpr int kRunSmemBytes = kRunStageVecs * kRunThreads * 16 + 128;   // 53,248 B of staging slots + the long-row list

// Long multi-run rows whose last run this CTA summed: all threads copy a block of consecutive run sums (they are
// contiguous in the partial buffer) into the staging memory, then the first lpr lanes of warp 0 add them in order.
// The fp32 add chain of a row is serial by definition; the copies are not, and 256 threads keep 52 KB in flight.
// Sum of the `nr` consecutive run sums at p, in order from +0, for column threadIdx.x (threads < lpr; others return 0).
// Called by every thread of the CTA.
__device__ __noinline__ float4 sum_long_row(const float* p, uint32_t nr, int D, int lpr, float4* stage) {
  const int chunk_rows = kRunStageVecs * kRunThreads / lpr;
  float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t c0 = 0; c0 < nr; c0 += chunk_rows) {
    const int cnt = (int)min((uint32_t)chunk_rows, nr - c0);
    const float* src = p + (int64_t)c0 * D;
    for (int idx = threadIdx.x; idx < cnt * lpr; idx += kRunThreads) cp_async16(stage + idx, src + (int64_t)idx * 4);
    cp_async_commit(); cp_async_wait<0>();
    __syncthreads();
    if ((int)threadIdx.x < lpr) {
      const float4* q = stage + threadIdx.x;
      int r = 0;
      for (; r + 8 <= cnt; r += 8) {
        float4 x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = q[(r + e) * lpr];
#pragma unroll
        for (int e = 0; e < 8; ++e) tot = add4(tot, x[e]);
      }
      for (; r < cnt; ++r) tot = add4(tot, q[r * lpr]);
    }
    __syncthreads();
  }
  return tot;
}

template <bool FUSED>
__device__ __forceinline__ void finish_long_rows(const ReduceArgs& a, float4* stage, const uint32_t* s_long, const uint32_t* s_nlong) {
  __syncthreads();                                   // every thread is past its last item; the list is complete
  const uint32_t n_long = min(*s_nlong, (uint32_t)kLongCap);
  if (n_long == 0) return;
  __threadfence();                                   // acquire side of the rows' completion counts
  for (uint32_t w = 0; w < n_long; ++w) {
    const uint4 info = __ldcg(a.mrow_info + s_long[w]);   // {row, runs, first run sum, count}
    const float4 tot = sum_long_row(a.partial + (int64_t)info.z * a.D, info.y, a.D, a.lpr, stage);
    if ((int)threadIdx.x < a.lpr) finish_row<FUSED>(a, info.x, (int)threadIdx.x, tot);
  }
}

// Every thread stages its own 16-byte pieces — up to 10 gradient rows and, for a single-run row, w, m, v — in shared
// memory with cp.async: the bytes in flight no longer occupy registers, so four CTAs fit an SM and each thread keeps
// up to 208 B outstanding.  A thread only reads back what it copied itself: cp.async.wait_group is the only wait.
template <bool FUSED, bool PREFETCH, bool PEER>
__global__ void __launch_bounds__(kRunThreads)
srm2_segment_runsum_kernel(ReduceArgs a) {
  extern __shared__ __align__(128) float4 stage[];                 // [kRunStageVecs][kRunThreads]
  uint32_t* s_long = reinterpret_cast<uint32_t*>(stage + kRunStageVecs * kRunThreads);   // behind the staging slots, so
  uint32_t& s_nlong = s_long[kLongCap];                                                  // that those stay 128-byte aligned
  if (threadIdx.x == 0) s_nlong = 0;
  __syncthreads();
  float4* mine = stage + threadIdx.x;
  const AdamSc sc = a.sc;
  const AdamFast fa = adam_fast_prepare(sc);
  const int64_t items = (int64_t)a.counters->n_runs * a.lpr;
  const int lane = threadIdx.x & 31;
  const unsigned gmask = a.lpr >= 32 ? 0xffffffffu : (((1u << a.lpr) - 1u) << (lane & ~(a.lpr - 1)));
  const int gleader = a.lpr >= 32 ? 0 : (lane & ~(a.lpr - 1));
  const int64_t stride = (int64_t)gridDim.x * kRunThreads;
  int64_t t = (int64_t)blockIdx.x * kRunThreads + threadIdx.x;
  auto split = [&](int64_t tt, int64_t& c, int& j4) {
    if (a.shift >= 0) { c = tt >> a.shift; j4 = (int)(tt & (a.lpr - 1)); } else { c = tt / a.lpr; j4 = (int)(tt - c * a.lpr); }
  };
  RunItem cur, nxt;
  int64_t c; int j4;
  if (PREFETCH && t < items) { split(t, c, j4); load_item(a, c, cur); }
  for (; t < items; t += stride) {
    split(t, c, j4);
    if (!PREFETCH) load_item(a, c, cur);
    const uint4 d = cur.d;
    const int len = (int)(d.y & 0xffu);
    const bool multi = (d.y & kMultiBit) != 0;
    // ---- all copies of this item ----
    float* b = nullptr;
    if (!multi) {
      const int64_t target = (int64_t)((uint64_t)d.z | ((uint64_t)d.w << 32));
      if (FUSED) {
        b = a.pool + target * (3 * (int64_t)a.D) + j4 * 4;
        cp_async16(mine + kRun * kRunThreads, b); cp_async16(mine + (kRun + 1) * kRunThreads, b + a.D);
        cp_async16(mine + (kRun + 2) * kRunThreads, b + 2 * a.D);
      } else {
        b = a.out + target * (int64_t)a.D + j4 * 4;
      }
    }
#pragma unroll
    for (int q = 0; q < kRun; ++q) {
      const uint32_t pos = (q & 1) ? cur.p[q / 2].y : cur.p[q / 2].x;
      if (q < len) cp_async16(mine + q * kRunThreads, grad_row<PEER>(a, pos) + j4 * 4);
    }
    cp_async_commit();
    if (PREFETCH && t + stride < items) { int64_t cn; int jn; split(t + stride, cn, jn); load_item(a, cn, nxt); }
    cp_async_wait<0>();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kRun; ++q)
      if (q < len) acc = add4(acc, mine[q * kRunThreads]);
    if (PREFETCH) cur = nxt;
    if (!multi) {
      const float4 g = add4(make_float4(0.f, 0.f, 0.f, 0.f), acc);
      if (FUSED) {
        float4 w = mine[kRun * kRunThreads], m = mine[(kRun + 1) * kRunThreads], v = mine[(kRun + 2) * kRunThreads];
        adam_vec4_fast(w, m, v, g, fa);
        *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
      } else {
        *reinterpret_cast<float4*>(b) = g;
      }
      continue;
    }
    float* pp = a.partial + (int64_t)d.z * a.D + j4 * 4;
    if (!a.inplace) { *reinterpret_cast<float4*>(pp) = acc; continue; }
    __stcg(reinterpret_cast<float4*>(pp), acc);
    __syncwarp(gmask);                                 // the group's stores are ordered before the leader's fence
    uint4 info = make_uint4(0u, 0u, 0u, 0u);
    if (lane == gleader) {
      info = __ldcg(reinterpret_cast<const uint4*>(a.mrow_info + d.w));
      __threadfence();                                 // release: the run sum is visible before the count
      const uint32_t old = atomicAdd(&a.mrow_info[d.w].w, 1u);
      info.w = old;
    }
    info.x = __shfl_sync(gmask, info.x, gleader); info.y = __shfl_sync(gmask, info.y, gleader);
    info.z = __shfl_sync(gmask, info.z, gleader); info.w = __shfl_sync(gmask, info.w, gleader);
    if (info.w != info.y - 1u) continue;               // not the last run of the row to finish
    if (info.y > (uint32_t)kInplaceMaxRuns) {          // a long row: left to the whole CTA, after its last item
      uint32_t slot = 0;
      if (lane == gleader) slot = atomicAdd(&s_nlong, 1u);
      slot = __shfl_sync(gmask, slot, gleader);
      if (slot < (uint32_t)kLongCap) { if (lane == gleader) s_long[slot] = d.w; continue; }
    }
    __threadfence();
    // the group that completes a row adds its run sums in order, staging kRun of them at a time the same way
    const float* p = a.partial + (int64_t)info.z * a.D + j4 * 4;
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r0 = 0; r0 < info.y; r0 += kRun) {
      const int cnt = (int)min((uint32_t)kRun, info.y - r0);
#pragma unroll
      for (int e = 0; e < kRun; ++e)
        if (e < cnt) cp_async16(mine + e * kRunThreads, p + (int64_t)(r0 + e) * a.D);
      cp_async_commit(); cp_async_wait<0>();
#pragma unroll
      for (int e = 0; e < kRun; ++e)
        if (e < cnt) tot = add4(tot, mine[e * kRunThreads]);
    }
    finish_row<FUSED>(a, info.x, j4, tot);
  }
  if (a.inplace) finish_long_rows<FUSED>(a, stage, s_long, &s_nlong);
}

// The same kernel for rows of 16 or 32 lanes (D = 64 or 128), where a run's lane group is an aligned half or whole warp
// with at least kRun lanes.  Differences that cut the instruction count by about a third:
//  - the positions of a run are held one per lane (lane q of the group holds position q) and broadcast with a shuffle
//    when row q is copied: one coalesced 40-byte load per run instead of ten loads per lane;
//  - a run of a single lookup carries its position in the descriptor and needs no position load at all;
//  - the copy and add loops run `len` times (len is uniform over the group) instead of ten predicated times;
//  - descriptors are fetched two items ahead and positions one item ahead, so neither is waited for.
template <bool FUSED, bool PEER>
__global__ void __launch_bounds__(kRunThreads, 4)
srm2_segment_runsum_wide_kernel(ReduceArgs a) {
  extern __shared__ __align__(128) float4 stage[];                 // [kRunStageVecs][kRunThreads]
  uint32_t* s_long = reinterpret_cast<uint32_t*>(stage + kRunStageVecs * kRunThreads);   // behind the staging slots, so
  uint32_t& s_nlong = s_long[kLongCap];                                                  // that those stay 128-byte aligned
  if (threadIdx.x == 0) s_nlong = 0;
  __syncthreads();
  float4* mine = stage + threadIdx.x;
  const AdamSc sc = a.sc;
  const AdamFast fa = adam_fast_prepare(sc);
  const int64_t items = (int64_t)a.counters->n_runs * a.lpr;
  const int lane = threadIdx.x & 31;
  const unsigned gmask = a.lpr >= 32 ? 0xffffffffu : (((1u << a.lpr) - 1u) << (lane & ~(a.lpr - 1)));
  const int gleader = a.lpr >= 32 ? 0 : (lane & ~(a.lpr - 1));
  const int gl = lane - gleader;                    // lane within the group
  const int64_t step = (int64_t)gridDim.x * kRunThreads;         // grid-stride: even waves whatever the number of runs
  int64_t t = (int64_t)blockIdx.x * kRunThreads + threadIdx.x;
  const int64_t end = items;
  const int j4 = (int)(t & (a.lpr - 1));
  auto run_of = [&](int64_t tt) { return tt >> a.shift; };
  auto load_desc = [&](int64_t tt) -> uint4 { return tt < end ? __ldg(a.run_desc + run_of(tt)) : make_uint4(0u, 0u, 0u, 0u); };
  auto load_pos = [&](const uint4& d, int64_t c) -> uint32_t {   // position gl of run c, for runs of more than one lookup
    const int len = (int)(d.y & 0xffu);
    return (len > 1 && gl < len) ? __ldg(a.run_pos + c * kRun + gl) : 0u;
  };
  auto lone = [](const uint4& d) { return d.y == 1u; };          // a row with a single lookup: one run of length one
  // descriptors of this item and the next two; positions of this item
  uint4 d0 = load_desc(t), d1 = load_desc(t + step), d2 = load_desc(t + 2 * step);
  uint32_t p0 = t < end ? load_pos(d0, run_of(t)) : 0u, p1 = 0;
  while (t < end) {
    if (FUSED && lone(d0) && lone(d1) && lone(d2)) {
      // ---- three single-lookup rows at once: 3 x (gradient row, w, m, v) = 12 of the 13 slots, 192 bytes in flight ----
      float* b0 = a.pool + (int64_t)((uint64_t)d0.z | ((uint64_t)d0.w << 32)) * (3 * (int64_t)a.D) + j4 * 4;
      float* b1 = a.pool + (int64_t)((uint64_t)d1.z | ((uint64_t)d1.w << 32)) * (3 * (int64_t)a.D) + j4 * 4;
      float* b2 = a.pool + (int64_t)((uint64_t)d2.z | ((uint64_t)d2.w << 32)) * (3 * (int64_t)a.D) + j4 * 4;
      cp_async16(mine, grad_row<PEER>(a, d0.x) + j4 * 4);
      cp_async16(mine + 4 * kRunThreads, grad_row<PEER>(a, d1.x) + j4 * 4);
      cp_async16(mine + 8 * kRunThreads, grad_row<PEER>(a, d2.x) + j4 * 4);
      cp_async16(mine + 1 * kRunThreads, b0); cp_async16(mine + 2 * kRunThreads, b0 + a.D); cp_async16(mine + 3 * kRunThreads, b0 + 2 * a.D);
      cp_async16(mine + 5 * kRunThreads, b1); cp_async16(mine + 6 * kRunThreads, b1 + a.D); cp_async16(mine + 7 * kRunThreads, b1 + 2 * a.D);
      cp_async16(mine + 9 * kRunThreads, b2); cp_async16(mine + 10 * kRunThreads, b2 + a.D); cp_async16(mine + 11 * kRunThreads, b2 + 2 * a.D);
      cp_async_commit();
      t += 3 * step;
      d0 = load_desc(t); d1 = load_desc(t + step); d2 = load_desc(t + 2 * step);
      cp_async_wait<0>();
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int e = 0; e < 3; ++e) {
        float* b = e == 0 ? b0 : (e == 1 ? b1 : b2);
        const float4 g = add4(zero, add4(zero, mine[(4 * e) * kRunThreads]));     // the run sum from +0, then the row sum from +0
        float4 w = mine[(4 * e + 1) * kRunThreads], m = mine[(4 * e + 2) * kRunThreads], v = mine[(4 * e + 3) * kRunThreads];
        adam_vec4_fast(w, m, v, g, fa);
        *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
      }
      if (t < end) p0 = load_pos(d0, run_of(t));
      continue;
    }
    const uint4 d = d0;
    const int len = (int)(d.y & 0xffu);
    const bool multi = (d.y & kMultiBit) != 0;
    // ---- copies of this item ----
    float* b = nullptr;
    if (!multi) {
      const int64_t target = (int64_t)((uint64_t)d.z | ((uint64_t)d.w << 32));
      if (FUSED) {
        b = a.pool + target * (3 * (int64_t)a.D) + j4 * 4;
        cp_async16(mine + kRun * kRunThreads, b); cp_async16(mine + (kRun + 1) * kRunThreads, b + a.D);
        cp_async16(mine + (kRun + 2) * kRunThreads, b + 2 * a.D);
      } else {
        b = a.out + target * (int64_t)a.D + j4 * 4;
      }
    }
    if (len == 1) {
      cp_async16(mine, grad_row<PEER>(a, d.x) + j4 * 4);
    } else {
      for (int q = 0; q < len; ++q) {
        const uint32_t pos = __shfl_sync(gmask, p0, gleader + q);
        cp_async16(mine + q * kRunThreads, grad_row<PEER>(a, pos) + j4 * 4);
      }
    }
    cp_async_commit();
    // ---- next items: descriptor three ahead, positions one ahead ----
    const uint4 d3 = load_desc(t + 3 * step);
    if (t + step < end) p1 = load_pos(d1, run_of(t + step));
    cp_async_wait<0>();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < len; ++q) acc = add4(acc, mine[q * kRunThreads]);
    d0 = d1; d1 = d2; d2 = d3; p0 = p1;
    t += step;
    if (!multi) {
      const float4 g = add4(make_float4(0.f, 0.f, 0.f, 0.f), acc);
      if (FUSED) {
        float4 w = mine[kRun * kRunThreads], m = mine[(kRun + 1) * kRunThreads], v = mine[(kRun + 2) * kRunThreads];
        adam_vec4_fast(w, m, v, g, fa);
        *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
      } else {
        *reinterpret_cast<float4*>(b) = g;
      }
      continue;
    }
    __stcg(reinterpret_cast<float4*>(a.partial + (int64_t)d.z * a.D + j4 * 4), acc);
    __syncwarp(gmask);                                 // the group's stores are ordered before the leader's fence
    uint4 info = make_uint4(0u, 0u, 0u, 0u);
    if (gl == 0) {
      info = __ldcg(reinterpret_cast<const uint4*>(a.mrow_info + d.w));
      __threadfence();                                 // release: the run sum is visible before the count
      info.w = atomicAdd(&a.mrow_info[d.w].w, 1u);
    }
    info.x = __shfl_sync(gmask, info.x, gleader); info.y = __shfl_sync(gmask, info.y, gleader);
    info.z = __shfl_sync(gmask, info.z, gleader); info.w = __shfl_sync(gmask, info.w, gleader);
    if (info.w != info.y - 1u) continue;               // not the last run of the row to finish
    if (info.y > (uint32_t)kInplaceMaxRuns) {          // a long row: left to the whole CTA, after its last item
      uint32_t slot = 0;
      if (lane == gleader) slot = atomicAdd(&s_nlong, 1u);
      slot = __shfl_sync(gmask, slot, gleader);
      if (slot < (uint32_t)kLongCap) { if (lane == gleader) s_long[slot] = d.w; continue; }
    }
    __threadfence();
    const float* p = a.partial + (int64_t)info.z * a.D + j4 * 4;
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r0 = 0; r0 < info.y; r0 += kRun) {
      const int cnt = (int)min((uint32_t)kRun, info.y - r0);
      for (int e = 0; e < cnt; ++e) cp_async16(mine + e * kRunThreads, p + (int64_t)(r0 + e) * a.D);
      cp_async_commit(); cp_async_wait<0>();
      for (int e = 0; e < cnt; ++e) tot = add4(tot, mine[e * kRunThreads]);
    }
    finish_row<FUSED>(a, info.x, j4, tot);
  }
  if (a.inplace) finish_long_rows<FUSED>(a, stage, s_long, &s_nlong);
}

// ------------------------------------------------------------------------------------------ multi-run rows

constexpr int kFinalWarps = 4;
constexpr int kFinalThreads = kFinalWarps * 32;
constexpr int kMaxColsPerLane = 4;                 // D <= 512
constexpr int kFinalSmemBytes = 64 * 1024;         // staging buffer of one CTA

// Adds `cnt` staged run sums (rows of lpr float4 in shared memory) to the running totals of this lane's columns.
__device__ __forceinline__ void add_staged(float4 (&tot)[kMaxColsPerLane], const float4* __restrict__ buf, int cnt, int lpr, int lane) {
#pragma unroll
  for (int q = 0; q < kMaxColsPerLane; ++q) {
    const int col = lane + 32 * q;
    if (col < lpr) {
      float4 t = tot[q];
      const float4* src = buf + col;
      int r = 0;
      for (; r + 8 <= cnt; r += 8) {
        float4 x[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] = src[(r + e) * lpr];
#pragma unroll
        for (int e = 0; e < 8; ++e) t = add4(t, x[e]);
      }
      for (; r < cnt; ++r) t = add4(t, src[r * lpr]);
      tot[q] = t;
    }
  }
}

// Multi-run rows: run sums added in order from +0.  A CTA takes four rows at a time.
//  - a row with at most `short_rows` run sums is handled by one warp: each lane copies its own 16-byte columns of all
//    run sums into shared memory with cp.async in one go (every load in flight at once) and adds them up;
//  - longer rows are then handled by the whole CTA, one after another: the run sums of a row are contiguous in the
//    partial buffer, so all threads copy a chunk of `chunk_rows` of them as one linear block, then warp 0 adds the
//    chunk (the fp32 add chain is the only serial part; a chunk of 128 rows is ~1 us of copy and ~0.3 us of adds).
template <bool FUSED>
__global__ void __launch_bounds__(kFinalThreads)
srm2_segment_final_kernel(ReduceArgs a, int short_rows, int chunk_rows) {
  extern __shared__ __align__(128) float4 smf[];                  // kFinalSmemBytes
  __shared__ uint32_t s_j[kFinalWarps], s_nr[kFinalWarps], s_pb[kFinalWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4* mine = smf + (size_t)warp * short_rows * a.lpr;
  const uint32_t n_mrows = a.counters->n_mrows;
  for (uint32_t g = blockIdx.x; g * kFinalWarps < n_mrows; g += gridDim.x) {
    const uint32_t mi = g * kFinalWarps + warp;
    uint32_t j = 0, nr = 0, pb = 0;
    if (mi < n_mrows) {
      j = a.mrows[mi];
      nr = (a.seg_end[j] - a.seg_start[j] + kRun - 1) / kRun;
      pb = a.bpre_m[j / kPlanThreads] + a.mrun_off[j];
    }
    if (lane == 0) { s_j[warp] = j; s_nr[warp] = nr; s_pb[warp] = pb; }
    if (nr > 0 && nr <= (uint32_t)short_rows) {
      const float* p = a.partial + (int64_t)pb * a.D;
      for (uint32_t r = 0; r < nr; ++r)
        for (int col = lane; col < a.lpr; col += 32) cp_async16(mine + (size_t)r * a.lpr + col, p + (int64_t)r * a.D + col * 4);
      cp_async_commit(); cp_async_wait<0>();
      float4 tot[kMaxColsPerLane];
#pragma unroll
      for (int q = 0; q < kMaxColsPerLane; ++q) tot[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      add_staged(tot, mine, (int)nr, a.lpr, lane);
#pragma unroll
      for (int q = 0; q < kMaxColsPerLane; ++q) { const int col = lane + 32 * q; if (col < a.lpr) finish_row<FUSED>(a, j, col, tot[q]); }
    }
    __syncthreads();
    for (int w = 0; w < kFinalWarps; ++w) {
      const uint32_t lnr = s_nr[w];
      if (lnr <= (uint32_t)short_rows) continue;       // uniform over the CTA
      const float* p = a.partial + (int64_t)s_pb[w] * a.D;
      float4 tot[kMaxColsPerLane];
#pragma unroll
      for (int q = 0; q < kMaxColsPerLane; ++q) tot[q] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (uint32_t c0 = 0; c0 < lnr; c0 += chunk_rows) {
        const int cnt = (int)min((uint32_t)chunk_rows, lnr - c0);
        const float* src = p + (int64_t)c0 * a.D;
        for (int idx = threadIdx.x; idx < cnt * a.lpr; idx += kFinalThreads) cp_async16(smf + idx, src + (int64_t)idx * 4);
        cp_async_commit(); cp_async_wait<0>();
        __syncthreads();
        if (warp == 0) add_staged(tot, smf, cnt, a.lpr, lane);
        __syncthreads();
      }
      if (warp == 0) {
#pragma unroll
        for (int q = 0; q < kMaxColsPerLane; ++q) { const int col = lane + 32 * q; if (col < a.lpr) finish_row<FUSED>(a, s_j[w], col, tot[q]); }
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------ small inputs
// One thread per (unique row, lane) walks the row's lookups in ascending position; lookups of the same 32-position
// window are summed from the first one, each window sum is then added to the row total (from +0).
template <bool FUSED>
__global__ void __launch_bounds__(256)
srm2_segment_windowed_kernel(ReduceArgs a) {
  const int64_t nu = load_nu(a.nu_host, a.nu_dev, a.cap);
  const int64_t items = nu * a.lpr;
  for (int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x; t < items; t += (int64_t)gridDim.x * 256) {
    int64_t j; int j4;
    if (a.shift >= 0) { j = t >> a.shift; j4 = (int)(t & (a.lpr - 1)); } else { j = t / a.lpr; j4 = (int)(t - j * a.lpr); }
    const uint32_t s0 = a.seg_start[j], s1 = a.seg_end[j];
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f), win = tot;
    uint32_t cur = 0xffffffffu;
    for (uint32_t i = s0; i < s1; ++i) {
      const uint32_t pos = a.spos[i];
      const float4 g = ld_stream4(a.grad + (int64_t)pos * a.D + j4 * 4);
      if (pos / kWindow != cur) {
        if (cur != 0xffffffffu) tot = add4(tot, win);
        cur = pos / kWindow; win = g;
      } else {
        win = add4(win, g);
      }
    }
    if (cur != 0xffffffffu) tot = add4(tot, win);
    finish_row<FUSED>(a, (uint32_t)j, j4, tot);
  }
}

// ------------------------------------------------------------------------------------------ host side
struct SegScratch {
  uint32_t *keyA, *valA, *keyB, *valB, *hist, *dtot, *seg_start, *seg_end, *run_off, *mrun_off, *mrow_off, *bsum_r, *bsum_m, *bsum_f, *mrows;
  uint4* run_desc; uint32_t* run_pos; uint4* mrow_info; SegCounters* counters; float* partial;
  int tiles, bits, passes, nblocks; char* zero; size_t zero_bytes;
};

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int ceil_log2(int64_t x) { int b = 0; while (((int64_t)1 << b) < x) ++b; return b; }

static size_t seg_layout(int64_t n, int64_t cap, int64_t D, char* base, SegScratch* s) {
  const int tiles = sort_tiles(n > 0 ? n : 1);
  const int keybits = ceil_log2(cap + 1 < 2 ? 2 : cap + 1);     // keys 0..cap (cap = invalid index)
  const int passes = (keybits + kMaxRadixBits - 1) / kMaxRadixBits;
  const int bits = (keybits + passes - 1) / passes;
  const int nblocks = (int)((cap + kPlanThreads - 1) / kPlanThreads);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t nn = (size_t)(n > 0 ? n : 1), cc = (size_t)(cap + 1), nb = (size_t)(nblocks + 1);
  const size_t o_ka = take(nn * 4), o_va = take(nn * 4), o_kb = take(nn * 4), o_vb = take(nn * 4);
  const size_t o_h = take(sort_hist_words(tiles, bits) * 4);
  // one zero-filled region per call: counters | digit totals | seg_start | seg_end
  const size_t zero_bytes = 256 + align_up(sort_dtot_words(tiles, bits, passes) * 4, 256) + cc * 4 * 2;
  const size_t o_z = take(zero_bytes);
  const size_t o_ct = o_z, o_dt = o_z + 256, o_ss = o_dt + align_up(sort_dtot_words(tiles, bits, passes) * 4, 256);
  const size_t o_ro = take(cc * 4), o_mo = take(cc * 4), o_fo = take(cc * 4);
  const size_t o_br = take(nb * 4), o_bm = take(nb * 4), o_bf = take(nb * 4);
  const size_t o_mr = take(cc * 4), o_rd = take(nn * 16), o_rp = take((nn * kRun + 16) * 4), o_mi = take((nn / (kRun + 1) + 2) * 16);
  const size_t max_partial = (size_t)(n / kRun + n / (kRun + 1) + 2);
  const size_t o_p = take(max_partial * (size_t)D * 4);
  if (s) {
    auto u = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    s->keyA = u(o_ka); s->valA = u(o_va); s->keyB = u(o_kb); s->valB = u(o_vb); s->hist = u(o_h); s->dtot = u(o_dt);
    s->seg_start = u(o_ss); s->seg_end = u(o_ss) + cc;
    s->run_off = u(o_ro); s->mrun_off = u(o_mo); s->mrow_off = u(o_fo); s->bsum_r = u(o_br); s->bsum_m = u(o_bm); s->bsum_f = u(o_bf);
    s->mrows = u(o_mr); s->run_desc = reinterpret_cast<uint4*>(base + o_rd); s->run_pos = u(o_rp); s->mrow_info = reinterpret_cast<uint4*>(base + o_mi); s->counters = reinterpret_cast<SegCounters*>(base + o_ct);
    s->partial = reinterpret_cast<float*>(base + o_p);
    s->tiles = tiles; s->bits = bits; s->passes = passes; s->nblocks = nblocks; s->zero = base + o_z; s->zero_bytes = zero_bytes;
  }
  return off;
}

// Launch of the run-sum kernel that fits the row width.
template <bool FUSED, bool PEER>
static int launch_runsum(const ReduceArgs& a, bool wide, int grid, cudaStream_t st) {
  if (wide) {
    if (note_cuda(cudaFuncSetAttribute(srm2_segment_runsum_wide_kernel<FUSED, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRunSmemBytes))) return SRM2_ERR_CUDA;
    srm2_segment_runsum_wide_kernel<FUSED, PEER><<<grid, kRunThreads, kRunSmemBytes, st>>>(a);
  } else {
    if (note_cuda(cudaFuncSetAttribute(srm2_segment_runsum_kernel<FUSED, kRunPrefetch, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRunSmemBytes))) return SRM2_ERR_CUDA;
    srm2_segment_runsum_kernel<FUSED, kRunPrefetch, PEER><<<grid, kRunThreads, kRunSmemBytes, st>>>(a);
  }
  return SRM2_OK;
}

struct PullSource { const float* const* peer_grad; int world; const uint32_t* src_code; };   // pull mode (fused, runs order only)

// phase bits: kSortPhase (radix passes) and kDescrPhase (boundaries, plan, run descriptors) together are the index half —
// everything that depends on the lookups' row indices only; kSumPhase = the kernels that read gradients and write rows.
// The parts of a split call communicate through the scratch buffer alone, so they may run on different streams (ordered
// by events), and the index work of later steps may run while the sum half of this one is still streaming.
constexpr int kSortPhase = 1, kSumPhase = 2, kDescrPhase = 4, kIndexPhase = kSortPhase | kDescrPhase, kAllPhases = 7;

static int segment_pipeline(bool fused, int order, const float* grad, const int64_t* inv, int64_t n, const int64_t* n_dev, int64_t D, int64_t nu_host,
                            const int64_t* nu_dev, int64_t cap, float* out, float* pool, const int64_t* slots,
                            const float* sc, void* scratch, size_t scratch_bytes, cudaStream_t st, const PullSource* pull = nullptr,
                            int phase = kAllPhases) {
  if (n < 0 || D <= 0 || cap < 0 || (nu_host < 0 && nu_dev == nullptr) || order < 0 || order > 2) return SRM2_ERR_ARG;
  if (nu_dev == nullptr) cap = nu_host;
  if (cap == 0) return SRM2_OK;
  const bool sort_phase = (phase & kSortPhase) != 0, descr_phase = (phase & kDescrPhase) != 0, sum_phase = (phase & kSumPhase) != 0;
  const bool index_phase = sort_phase || descr_phase;
  if (n > 0 && ((sum_phase && grad == nullptr && pull == nullptr) || (sort_phase && inv == nullptr))) return SRM2_ERR_ARG;
  if (phase != kAllPhases && (!fused || order != SRM2_ORDER_RUNS)) return SRM2_ERR_ARG;
  if (pull) {
    if (!fused || order != SRM2_ORDER_RUNS || pull->world < 1 || pull->world > kMaxGradPeers || (sum_phase && pull->peer_grad == nullptr) ||
        (descr_phase && pull->src_code == nullptr))
      return SRM2_ERR_ARG;
    for (int r = 0; sum_phase && r < pull->world; ++r)
      if (pull->peer_grad[r] == nullptr || !aligned16(pull->peer_grad[r])) return SRM2_ERR_ARG;
  }
  if (fused ? (slots == nullptr || (sum_phase && (pool == nullptr || sc == nullptr))) : out == nullptr) return SRM2_ERR_ARG;
  // n < 2^21: the plan kernel scans three run counters packed into 21-bit fields of one word
  if ((D & 3) != 0 || D > 128 * kMaxColsPerLane || n >= ((int64_t)1 << 21) || cap >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (sum_phase && ((n > 0 && !pull && !aligned16(grad)) || (fused ? !aligned16(pool) : !aligned16(out)))) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < seg_layout(n, cap, D, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  SegScratch s;
  seg_layout(n, cap, D, static_cast<char*>(scratch), &s);
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  const bool small = order == SRM2_ORDER_WINDOWS || (order == SRM2_ORDER_AUTO && n <= kSmallN);
  int launches = 0;

  // empty ranges for rows that no lookup names; counters (incl. the finished-CTA count) start at zero
  if (sort_phase && note_cuda(cudaMemsetAsync(s.zero, 0, s.zero_bytes, st))) return SRM2_ERR_CUDA;
  // 1. sort (key = inv, value = position), 2. boundaries
  const uint32_t *skey = (s.passes & 1) ? s.keyA : s.keyB, *spos = (s.passes & 1) ? s.valA : s.valB;   // where the last pass lands
  if (n > 0 && sort_phase) {
    SortBuffers sb{s.keyA, s.valA, s.keyB, s.valB, s.hist, s.dtot, s.tiles};
    const uint32_t* hb = nullptr;
    const int rc = radix_sort_by_key(inv, n, n_dev, /*mod=*/0, cap, s.bits, s.passes, sb, &skey, &spos, &hb, &launches, st);
    if (rc != SRM2_OK) return rc;
  }
  if (n > 0 && descr_phase) {
    srm2_segment_bounds_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(skey, n, n_dev, s.seg_start, s.seg_end, cap);
    ++launches;
  }
  ReduceArgs a{};
  a.grad = grad; a.D = (int)D; a.lpr = lpr; a.shift = shift; a.skey = skey; a.spos = spos; a.seg_start = s.seg_start; a.seg_end = s.seg_end;
  a.run_desc = s.run_desc; a.run_pos = s.run_pos; a.mrows = s.mrows; a.mrow_info = s.mrow_info; a.counters = s.counters;
  a.inplace = (lpr <= 32 && (lpr & (lpr - 1)) == 0) ? 1 : 0; a.mrun_off = s.mrun_off; a.bpre_m = s.bsum_m; a.partial = s.partial;
  a.out = out; a.pool = pool; a.slots = slots;
  if (fused && sum_phase) a.sc = AdamSc{sc[0], sc[1], sc[2], sc[3], sc[4], sc[5], sc[6], sc[7]};
  a.nu_host = nu_host; a.nu_dev = nu_dev; a.cap = cap; a.n = n;
  if (pull && sum_phase) for (int r = 0; r < pull->world; ++r) a.peer[r] = pull->peer_grad[r];
  if (small) {
    const int64_t row_items = cap * lpr;
    const int grid_rows = (int)((row_items + 255) / 256 < (int64_t)kSMs * 16 ? (row_items + 255) / 256 : (int64_t)kSMs * 16);
    stage_begin(st);
    if (fused) srm2_segment_windowed_kernel<true><<<grid_rows, 256, 0, st>>>(a);
    else srm2_segment_windowed_kernel<false><<<grid_rows, 256, 0, st>>>(a);
    stage_end(st);
    return launch_status(launches + 1);
  }
  // 3. plan, 4. descriptors.  A split call leaves rows without lookups alone (its index half must not write rows).
  if (sort_phase && !descr_phase && !sum_phase) return launch_status(launches);
  if (descr_phase) {
    const int skip_empty = phase != kAllPhases;
    if (fused)
      srm2_segment_plan_kernel<true><<<s.nblocks, kPlanThreads, 0, st>>>(a, s.run_off, s.mrun_off, s.mrow_off, s.bsum_r, s.bsum_m, s.bsum_f,
                                                                        s.counters, s.nblocks, skip_empty);
    else
      srm2_segment_plan_kernel<false><<<s.nblocks, kPlanThreads, 0, st>>>(a, s.run_off, s.mrun_off, s.mrow_off, s.bsum_r, s.bsum_m, s.bsum_f,
                                                                         s.counters, s.nblocks, skip_empty);
    if (n > 0)
      srm2_segment_descr_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(skey, spos, n, n_dev, s.seg_start, s.seg_end, s.run_off, s.mrun_off, s.mrow_off,
                                                                            s.bsum_r, s.bsum_m, s.bsum_f, s.counters, fused ? slots : nullptr, pull ? pull->src_code : nullptr, s.run_desc, s.run_pos, s.mrows, s.mrow_info,
                                                                            nu_host, nu_dev, cap);
    launches += n > 0 ? 2 : 1;
    if (!sum_phase) return launch_status(launches);
  }
  // 5. run sums, 6. multi-run rows
  const int64_t run_items_max = n * lpr;
  // One-call form: two waves of CTAs that loop over the runs.  Split form: the sum half shares the GPU with other streams'
  // small kernels (the next steps' index work), so it is cut into many short-lived CTAs — SM room frees up every few
  // microseconds and the block scheduler hands it to whichever stream has work.
  const int64_t cta_cap = (int64_t)kSMs * (phase == kSumPhase ? 32 : 8);
  const int grid_runs = (int)((run_items_max + 255) / 256 < cta_cap ? (run_items_max + 255) / 256 : cta_cap);
  const int rows_fit = (int)(kFinalSmemBytes / (D * 4));                 // run sums that fit the CTA's staging buffer
  const int short_rows = rows_fit / kFinalWarps, chunk_rows = rows_fit;
  const size_t sm_final = kFinalSmemBytes;
  const int64_t groups_max = (n / (kRun + 1) + kFinalWarps) / kFinalWarps;
  const int grid_final = (int)(groups_max < (int64_t)kSMs * 3 ? groups_max : (int64_t)kSMs * 3);
  const bool wide = (lpr == 16 || lpr == 32);            // a run's lanes are an aligned half or whole warp of >= kRun lanes
  stage_begin(st);
  if (n > 0) {
    int rc;
    if (fused) rc = pull ? launch_runsum<true, true>(a, wide, grid_runs, st) : launch_runsum<true, false>(a, wide, grid_runs, st);
    else rc = launch_runsum<false, false>(a, wide, grid_runs, st);
    if (rc != SRM2_OK) return rc;
    if (!a.inplace) {
      if (fused) {
        if (note_cuda(cudaFuncSetAttribute(srm2_segment_final_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_final))) return SRM2_ERR_CUDA;
        srm2_segment_final_kernel<true><<<grid_final, kFinalThreads, sm_final, st>>>(a, short_rows, chunk_rows);
      } else {
        if (note_cuda(cudaFuncSetAttribute(srm2_segment_final_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_final))) return SRM2_ERR_CUDA;
        srm2_segment_final_kernel<false><<<grid_final, kFinalThreads, sm_final, st>>>(a, short_rows, chunk_rows);
      }
    }
  }
  stage_end(st);
  return launch_status(launches + (n > 0 ? (a.inplace ? 1 : 2) : 0));
}

}  // namespace srm2

extern "C" size_t srm2_segment_scratch_bytes(int64_t n, int64_t max_unique, int64_t D) {
  if (n < 0 || max_unique < 0 || D <= 0) return 0;
  return srm2::seg_layout(n, max_unique, D, nullptr, nullptr);
}

extern "C" int srm2_segment_reduce_f32(const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t n_unique,
                                       const int64_t* n_unique_dev, int64_t max_unique, int order, float* out, void* scratch,
                                       size_t scratch_bytes, srm2_stream_t stream) {
  return srm2::segment_pipeline(false, order, grad, inv, n, nullptr, D, n_unique, n_unique_dev, max_unique, out, nullptr, nullptr, nullptr,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int srm2_reduce_adam_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n,
                                    int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique,
                                    int order, const float sc[8], void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  return srm2::segment_pipeline(true, order, grad, inv, n, nullptr, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc, scratch,
                                scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int srm2_reduce_adam_pull_f32(float* pool, const int64_t* slots, const float* const* peer_grad, int64_t world,
                                         const uint32_t* src_code, const int64_t* inv, int64_t n, const int64_t* n_dev, int64_t D,
                                         int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, const float sc[8],
                                         void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  if (peer_grad == nullptr || world < 1 || world > srm2::kMaxGradPeers) return SRM2_ERR_ARG;
  const srm2::PullSource pull{peer_grad, (int)world, src_code};
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, nullptr, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), &pull);
}

extern "C" int srm2_reduce_adam_index(const int64_t* slots, const uint32_t* src_code, const int64_t* inv, int64_t n, const int64_t* n_dev,
                                      int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, int part, void* scratch,
                                      size_t scratch_bytes, srm2_stream_t stream) {
  if (part < 0 || part > 2) return SRM2_ERR_ARG;
  const srm2::PullSource pull{nullptr, 1, src_code};
  const int phase = part == SRM2_INDEX_SORT ? srm2::kSortPhase : (part == SRM2_INDEX_DESCRIPTORS ? srm2::kDescrPhase : srm2::kIndexPhase);
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, nullptr, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, nullptr, slots, nullptr,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), src_code ? &pull : nullptr, phase);
}

extern "C" int srm2_reduce_adam_apply_f32(float* pool, const int64_t* slots, const float* grad, const float* const* peer_grad, int64_t world,
                                          int64_t n, const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev,
                                          int64_t max_unique, const float sc[8], void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  if ((grad == nullptr) == (peer_grad == nullptr) && n > 0) return SRM2_ERR_ARG;       // exactly one gradient source
  if (peer_grad != nullptr && (world < 1 || world > srm2::kMaxGradPeers)) return SRM2_ERR_ARG;
  const srm2::PullSource pull{peer_grad, (int)world, nullptr};
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, grad, nullptr, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), peer_grad ? &pull : nullptr, srm2::kSumPhase);
}

extern "C" int srm2_reduce_adam_nd_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n,
                                       const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev,
                                       int64_t max_unique, int order, const float sc[8], void* scratch, size_t scratch_bytes,
                                       srm2_stream_t stream) {
  return srm2::segment_pipeline(true, order, grad, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}
