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
//   3. plan.  The work item is a CHUNK: up to kChunkRuns consecutive runs (60 lookups) of one row.
//        rows of one chunk      : the row is its own item (nothing to prepare: the run-sum kernel reads the row's segment
//                                 bounds); it does everything — run sums, their sum, the row's Adam update (or store);
//        longer rows ("long")   : several items.  The first chunk adds its run sums locally and leaves one partial vector
//                                 (the sum so far); every later chunk leaves one partial vector per run.  A row's partials
//                                 are contiguous and in order, so the row total is their left-to-right sum from +0 —
//                                 exactly the order above.  One thread per row: a long row takes its range of chunk
//                                 descriptors and of partial slots from two counters (atomics; which range a row gets
//                                 does not matter, the order inside a row is fixed by the layout) and writes the
//                                 descriptors.  No scan, no second kernel.
//      Long rows' chunks come first in item order, so their partials are ready while the bulk is still streaming.
//   4. run sums: an aligned group of D/4 lanes per item streams the item's gradient rows through per-thread shared
//      memory slots with cp.async — five rows in flight while the previous five are added — so a 60-lookup item never
//      waits for more than its first loads.  One release (fence + counter increment) per chunk of a long row; the chunk
//      that completes a row adds the row's partials (a rolling window of twelve in flight; rows with many partials are
//      left to the whole CTA, which copies ~50 of them at a time into shared memory, double-buffered) and finishes it.
// Gradient rows are read exactly once (D*4 bytes per lookup); everything else is small integer traffic.
#include "common.cuh"
#include "exact.cuh"
#include "peer.cuh"
#include "scan.cuh"
#include "sort.cuh"

namespace srm2 {

constexpr int kRun = 10;            // lookups per run (large inputs)
constexpr int kChunkRuns = 6;       // runs per work item
constexpr int kChunk = kRun * kChunkRuns;
constexpr int kSmallN = 3072;       // inputs up to this many lookups use the windowed order
constexpr int kWindow = 32;
constexpr int kPlanThreads = 256;

struct SegCounters { uint32_t n_lchunks, n_lrows, n_parts; };
constexpr int kMaxGradPeers = 16;
constexpr int kPeerShift = 24;      // pull mode: a lookup is named by (source rank << 24) | row in that rank's gradient buffer
// Pull mode with sums prepared at the source (srm2_presum_request): a name with kOutBit set is a row of the source rank's
// buffer of prepared sums instead of its gradient buffer; kSkipName marks a lookup whose gradient is part of such a sum.
constexpr uint32_t kOutBit = 0x800000u, kSkipName = 0xffffffffu;
constexpr int kReqWords = 12;       // a request: {number of rows m, their positions [10], unused}

struct ReduceArgs {
  const float* grad; int D; int lpr; int shift;
  const uint32_t* skey; const uint32_t* spos; const uint32_t* seg_start; const uint32_t* seg_end;
  const uint4* chunk_desc; const uint4* row_desc; const uint32_t* pos_sorted; uint4* lrow_info; const SegCounters* counters; int inplace;
  float* partial;
  float* out;                                     // [nu, D] (unfused) or nullptr
  float* pool; const int64_t* slots; AdamSc sc;   // fused Adam: pool [C,3,D], slots[j] = pool row of unique row j
  int64_t nu_host; const int64_t* nu_dev; int64_t cap; int64_t n;
  const float* peer[kMaxGradPeers];               // pull mode: gradient buffers of all ranks (peer pointers), see grad_row
  const float* peer_out[kMaxGradPeers];           // ... and their buffers of prepared sums (this rank's region), or unused
  const uint32_t* err;                            // pull mode: status word of the exchange, or nullptr; non-zero: touch nothing
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
  if (PEER) {
    const uint32_t r = code >> kPeerShift;
    if (code & kOutBit) return a.peer_out[r] + (int64_t)(code & (kOutBit - 1u)) * a.D;
    return a.peer[r] + (int64_t)(code & (kOutBit - 1u)) * a.D;
  }
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
// In pull mode the kernel also leaves, at every sorted index, the name of the lookup's gradient row ((rank, row) code).
__global__ void __launch_bounds__(256)
srm2_segment_bounds_kernel(const uint32_t* __restrict__ skey, const uint32_t* __restrict__ spos, int64_t n_host,
                           const int64_t* __restrict__ n_dev, uint32_t* __restrict__ seg_start, uint32_t* __restrict__ seg_end,
                           int64_t cap, const uint32_t* __restrict__ src_code, uint32_t* __restrict__ names) {
  const int64_t n = eff_count(n_host, n_dev);
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    if (src_code) names[i] = src_code[spos[i]];
    const uint32_t k = skey[i];
    if ((int64_t)k >= cap) continue;
    if (i == 0 || skey[i - 1] != k) seg_start[k] = (uint32_t)i;
    if (i == n - 1 || skey[i + 1] != k) seg_end[k] = (uint32_t)(i + 1);
  }
}

// ------------------------------------------------------------------------------------------ plan
// What a row of `len` lookups needs.
struct RowShape { uint32_t runs, chunks, parts; bool is_long; };
__device__ __forceinline__ RowShape row_shape(uint32_t len) {
  RowShape r;
  r.runs = (len + kRun - 1) / kRun; r.chunks = (r.runs + kChunkRuns - 1) / kChunkRuns; r.is_long = r.chunks > 1;
  r.parts = r.is_long ? 1u + r.runs - (uint32_t)kChunkRuns : 0u;      // the first chunk's sum, then one per later run
  return r;
}

// One thread per unique row.  Rows without lookups are finished here (zero gradient).  A long row takes `chunks`
// consecutive chunk descriptors, `parts` consecutive partial slots and one entry of lrow_info, and fills them in:
//   row_desc[j]   = the row's own item (see below)
//   chunk_desc[c] = {sorted index of the chunk's first lookup, L | kLongBit (| kFirstBit for the row's first chunk),
//                    first partial slot the chunk writes, index of the row in lrow_info};  L = lookups of the chunk
//   lrow_info[w]  = {unique row, number of runs, first partial slot, finished-chunk counter = 0}
constexpr uint32_t kLongBit = 0x80000000u, kFirstBit = 0x40000000u;
template <bool FUSED>
__global__ void __launch_bounds__(kPlanThreads)
srm2_segment_plan_kernel(ReduceArgs a, uint4* __restrict__ chunk_desc, uint4* __restrict__ row_desc, SegCounters* __restrict__ counters,
                         int skip_empty) {
  const int64_t nu = load_nu(a.nu_host, a.nu_dev, a.cap);
  for (int64_t j = (int64_t)blockIdx.x * kPlanThreads + threadIdx.x; j < nu; j += (int64_t)gridDim.x * kPlanThreads) {
    const uint32_t s = a.seg_start[j], len = a.seg_end[j] - s;
    const RowShape r = row_shape(len);
    // the row's own item: {sorted index of its first lookup — or, for a single lookup, that lookup's name —, number of
    // lookups (0: nothing to do under this entry), 64-bit target: the pool row (fused) or the row index}
    const uint64_t target = FUSED ? (uint64_t)a.slots[j] : (uint64_t)j;
    row_desc[j] = make_uint4(len == 1 ? a.pos_sorted[s] : s, (len == 0 || r.is_long) ? 0u : len, (uint32_t)target, (uint32_t)(target >> 32));
    if (len == 0) {
      if (!skip_empty)
        for (int j4 = 0; j4 < a.lpr; ++j4) finish_row<FUSED>(a, (uint32_t)j, j4, make_float4(0.f, 0.f, 0.f, 0.f));
      continue;
    }
    if (!r.is_long) continue;
    const uint32_t c0 = atomicAdd(&counters->n_lchunks, r.chunks);
    const uint32_t base = atomicAdd(&counters->n_parts, r.parts);
    const uint32_t mi = atomicAdd(&counters->n_lrows, 1u);
    a.lrow_info[mi] = make_uint4((uint32_t)j, r.runs, base, 0u);
    for (uint32_t q = 0; q < r.chunks; ++q) {
      const uint32_t first = s + q * (uint32_t)kChunk, L = min((uint32_t)kChunk, len - q * (uint32_t)kChunk);
      const uint32_t slot = q == 0 ? base : base + 1u + (q - 1u) * (uint32_t)kChunkRuns;
      chunk_desc[c0 + q] = make_uint4(first, L | kLongBit | (q == 0 ? kFirstBit : 0u), slot, mi);
    }
  }
}

// ------------------------------------------------------------------------------------------ run sums
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Stages this lane's 16 bytes of a lookup's gradient row.  A lookup whose gradient went into a sum prepared at its source
// contributes +0 instead (the running sum of a run starts at +0 and is therefore never -0, so adding +0 leaves it as it is).
template <bool PEER>
__device__ __forceinline__ void stage_lookup(const ReduceArgs& a, float4* slot, uint32_t name, int j4) {
  if (PEER && name == kSkipName) *slot = make_float4(0.f, 0.f, 0.f, 0.f);
  else cp_async16(slot, grad_row<PEER>(a, name) + j4 * 4);
}

constexpr int kRunThreads = 128;
constexpr int kRunStageVecs = kRun + 3;                                  // gradient rows + w, m, v
constexpr int kWarpChainMax = 96;         // rows with more partial vectors are added up by a whole CTA (below)
constexpr int kLongCap = 16;              // such rows one CTA can take over; further ones are finished by their lane group
constexpr int kRunSmemBytes = kRunStageVecs * kRunThreads * 16 + 128;   // 26,624 B of staging slots + the long-row list

// Sum of `n` consecutive partial vectors at p (this lane's 16 bytes of each), in order from +0: twelve slots as three
// groups of four, the oldest group is added while the two younger ones are in flight.
__device__ __forceinline__ float4 chain_ring(const float* p, uint32_t n, int D, float4* mine) {
  float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
  auto issue = [&](uint32_t first, int grp) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (first + e < n) cp_async16(mine + (grp * 4 + e) * kRunThreads, p + (int64_t)(first + e) * D);
    cp_async_commit();
  };
  issue(0, 0); issue(4, 1); issue(8, 2);
  int grp = 0;
  for (uint32_t k = 0; k < n; k += 4) {
    cp_async_wait<2>();
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (k + e < n) tot = add4(tot, mine[(grp * 4 + e) * kRunThreads]);
    issue(k + 12, grp);
    grp = grp == 2 ? 0 : grp + 1;
  }
  cp_async_wait<0>();
  return tot;
}

// Rows with many partial vectors, by the whole CTA: all threads copy a block of consecutive partials (they are
// contiguous) into one half of the staging memory while the first lpr threads add the block in the other half.  The
// fp32 add chain of a row is serial by definition; the copies are not.  Called by every thread; threads >= lpr return 0.
__device__ __noinline__ float4 sum_long_row(const float* p, uint32_t nr, int D, int lpr, float4* stage) {
  const int half_rows = (kRunStageVecs * kRunThreads / lpr) / 2;
  auto issue = [&](uint32_t c0, int buf) {
    if (c0 < nr) {
      const int cnt = (int)min((uint32_t)half_rows, nr - c0);
      const float* src = p + (int64_t)c0 * D;
      float4* dst = stage + (size_t)buf * half_rows * lpr;
      for (int idx = threadIdx.x; idx < cnt * lpr; idx += kRunThreads) cp_async16(dst + idx, src + (int64_t)idx * 4);
    }
    cp_async_commit();
  };
  float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
  issue(0, 0);
  int buf = 0;
  for (uint32_t c0 = 0; c0 < nr; c0 += half_rows) {
    issue(c0 + half_rows, buf ^ 1);
    cp_async_wait<1>();
    __syncthreads();
    if ((int)threadIdx.x < lpr) {
      const int cnt = (int)min((uint32_t)half_rows, nr - c0);
      const float4* q = stage + (size_t)buf * half_rows * lpr + threadIdx.x;
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
    buf ^= 1;
  }
  cp_async_wait<0>();
  return tot;
}

__device__ __forceinline__ uint32_t parts_of(uint32_t runs) { return 1u + runs - (uint32_t)kChunkRuns; }

template <bool FUSED>
__device__ __forceinline__ void finish_long_rows(const ReduceArgs& a, float4* stage, const uint32_t* s_long, const uint32_t* s_nlong) {
  __syncthreads();                                   // every thread is past its last item; the list is complete
  const uint32_t n_long = min(*s_nlong, (uint32_t)kLongCap);
  if (n_long == 0) return;
  __threadfence();                                   // acquire side of the rows' completion counts
  for (uint32_t w = 0; w < n_long; ++w) {
    const uint4 info = __ldcg(a.lrow_info + s_long[w]);   // {row, runs, first partial, count}
    const float4 tot = sum_long_row(a.partial + (int64_t)info.z * a.D, parts_of(info.y), a.D, a.lpr, stage);
    if ((int)threadIdx.x < a.lpr) finish_row<FUSED>(a, info.x, (int)threadIdx.x, tot);
  }
}

// Rows of 16 or 32 lanes (D = 64 or 128): an item's lane group is an aligned half or whole warp with at least kRun lanes.
//  - the names of a run's gradient rows are held one per lane (lane q holds row q) and broadcast with a shuffle when row
//    q is copied: one coalesced 40-byte load per run; a row of a single lookup carries its name in the descriptor;
//  - three rows of a single lookup each are handled at once (12 of the 13 slots, 192 bytes per thread in flight);
//  - a one-run item issues all its copies at once; longer items stream run after run through two half-run slot sets;
//  - descriptors are fetched two items ahead and the first run's names one item ahead, so neither is waited for.
template <bool FUSED, bool PEER>
__global__ void __launch_bounds__(kRunThreads, 8)
srm2_segment_runsum_wide_kernel(ReduceArgs a) {
  extern __shared__ __align__(128) float4 stage[];                 // [kRunStageVecs][kRunThreads]
  uint32_t* s_long = reinterpret_cast<uint32_t*>(stage + kRunStageVecs * kRunThreads);   // behind the staging slots, so
  uint32_t& s_nlong = s_long[kLongCap];                                                  // that those stay 128-byte aligned
  uint32_t& s_stop = s_long[kLongCap + 1];
  if (threadIdx.x == 0) {
    s_nlong = 0;
    if (PEER) s_stop = a.err != nullptr ? *reinterpret_cast<const volatile uint32_t*>(a.err) : 0u;
  }
  __syncthreads();
  if (PEER && s_stop != 0u) return;                  // the exchange of this (or an earlier) step failed: the shard stays as it is
  float4* mine = stage + threadIdx.x;
  const AdamSc sc = a.sc;
  const AdamFast fa = adam_fast_prepare(sc);
  // items: the long rows' chunks (descriptors), then every unique row (its segment bounds are its descriptor; long rows
  // and rows without lookups come out as L = 0 and are skipped)
  const int64_t n_lchunks = a.counters->n_lchunks;
  const int64_t items = (n_lchunks + load_nu(a.nu_host, a.nu_dev, a.cap)) * a.lpr;
  const int lane = threadIdx.x & 31;
  const unsigned gmask = a.lpr >= 32 ? 0xffffffffu : (((1u << a.lpr) - 1u) << (lane & ~(a.lpr - 1)));
  const int gleader = a.lpr >= 32 ? 0 : (lane & ~(a.lpr - 1));
  const int gl = lane - gleader;                    // lane within the group
  const int64_t step = (int64_t)gridDim.x * kRunThreads;         // grid-stride: even waves whatever the number of items
  int64_t t = (int64_t)blockIdx.x * kRunThreads + threadIdx.x;
  const int64_t end = items;
  const int j4 = (int)(t & (a.lpr - 1));
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  // descriptor of item tt: {x = sorted index of the first lookup, y = L | flags, (z, w) = target row / (slot, long row)}
  auto load_desc = [&](int64_t tt) -> uint4 {
    if (tt >= end) return make_uint4(0u, 0u, 0u, 0u);
    const int64_t c = tt >> a.shift;
    return c < n_lchunks ? __ldg(a.chunk_desc + c) : __ldg(a.row_desc + (c - n_lchunks));
  };
  auto lookups = [](const uint4& d) { return (int)(d.y & 0xffu); };
  auto lone = [](const uint4& d) { return d.y == 1u; };          // a row with a single lookup
  // names of the first run of an item (lane gl holds row gl); a single lookup carries its name in the descriptor
  auto first_names = [&](const uint4& d) -> uint32_t {
    const int L = lookups(d);
    if (lone(d)) return d.x;
    return gl < min(L, kRun) ? __ldg(a.pos_sorted + d.x + gl) : 0u;
  };
  uint4 d0 = load_desc(t), d1 = load_desc(t + step), d2 = load_desc(t + 2 * step);
  uint32_t p0 = first_names(d0);
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
#pragma unroll
      for (int e = 0; e < 3; ++e) {
        float* b = e == 0 ? b0 : (e == 1 ? b1 : b2);
        const float4 g = add4(zero, add4(zero, mine[(4 * e) * kRunThreads]));     // the run sum from +0, then the row sum from +0
        float4 w = mine[(4 * e + 1) * kRunThreads], m = mine[(4 * e + 2) * kRunThreads], v = mine[(4 * e + 3) * kRunThreads];
        adam_vec4_fast(w, m, v, g, fa);
        *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
      }
      p0 = first_names(d0);
      continue;
    }
    const uint4 d = d0;
    const int L = lookups(d);
    const bool is_long = (d.y & kLongBit) != 0, is_first = (d.y & kFirstBit) != 0;
    const uint32_t names0 = p0;
    // descriptors of the next items and the names of the next item's first run, before this item's work
    d0 = d1; d1 = d2; d2 = load_desc(t + 3 * step);
    p0 = first_names(d0);
    t += step;
    if (L == 0) continue;                              // a long row's own entry (its chunks are items of their own), or no lookups
    float* b = nullptr;
    if (!is_long) {
      const int64_t target = (int64_t)((uint64_t)d.z | ((uint64_t)d.w << 32));
      if (FUSED) {
        b = a.pool + target * (3 * (int64_t)a.D) + j4 * 4;
        cp_async16(mine + kRun * kRunThreads, b); cp_async16(mine + (kRun + 1) * kRunThreads, b + a.D);
        cp_async16(mine + (kRun + 2) * kRunThreads, b + 2 * a.D);
      } else {
        b = a.out + target * (int64_t)a.D + j4 * 4;
      }
    }
    float4 total = zero;
    if (L <= kRun) {
      // ---- one run: every copy at once ----
      for (int q = 0; q < L; ++q) {
        const uint32_t pos = __shfl_sync(gmask, names0, gleader + q);
        stage_lookup<PEER>(a, mine + q * kRunThreads, pos, j4);
      }
      cp_async_commit();
      cp_async_wait<0>();
      float4 acc = zero;
      for (int q = 0; q < L; ++q) acc = add4(acc, mine[q * kRunThreads]);
      if (is_long && !is_first) __stcg(reinterpret_cast<float4*>(a.partial + (int64_t)d.z * a.D + j4 * 4), acc);
      else total = add4(zero, acc);
    } else {
      // ---- several runs: half a run in flight while the other half is added ----
      const int nruns = (L + kRun - 1) / kRun;
      uint32_t names = names0;
      auto issue_half = [&](uint32_t nm, int len_r, int h) {       // rows [5h, 5h+5) of a run of len_r rows
#pragma unroll
        for (int q = 0; q < kRun / 2; ++q) {
          const uint32_t pos = __shfl_sync(gmask, nm, gleader + h * (kRun / 2) + q);
          if (h * (kRun / 2) + q < len_r) stage_lookup<PEER>(a, mine + (h * (kRun / 2) + q) * kRunThreads, pos, j4);
        }
        cp_async_commit();
      };
      issue_half(names, min(L, kRun), 0);
      issue_half(names, min(L, kRun), 1);
      for (int r = 0; r < nruns; ++r) {
        const int len_r = min(kRun, L - r * kRun), len_n = min(kRun, L - (r + 1) * kRun);     // len_n <= 0: no next run
        const uint32_t next = (r + 1 < nruns && gl < len_n) ? __ldg(a.pos_sorted + d.x + (r + 1) * kRun + gl) : 0u;
        cp_async_wait<1>();
        float4 acc = zero;
#pragma unroll
        for (int q = 0; q < kRun / 2; ++q)
          if (q < len_r) acc = add4(acc, mine[q * kRunThreads]);
        issue_half(next, len_n, 0);
        cp_async_wait<1>();
#pragma unroll
        for (int q = kRun / 2; q < kRun; ++q)
          if (q < len_r) acc = add4(acc, mine[q * kRunThreads]);
        issue_half(next, len_n, 1);
        if (is_long && !is_first) __stcg(reinterpret_cast<float4*>(a.partial + (int64_t)(d.z + r) * a.D + j4 * 4), acc);
        else total = add4(total, acc);
      }
      cp_async_wait<0>();
    }
    if (!is_long) {
      if (FUSED) {
        float4 w = mine[kRun * kRunThreads], m = mine[(kRun + 1) * kRunThreads], v = mine[(kRun + 2) * kRunThreads];
        adam_vec4_fast(w, m, v, total, fa);
        *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
      } else {
        *reinterpret_cast<float4*>(b) = total;
      }
      continue;
    }
    if (is_first) __stcg(reinterpret_cast<float4*>(a.partial + (int64_t)d.z * a.D + j4 * 4), total);
    __syncwarp(gmask);                                 // the group's stores are ordered before the leader's fence
    uint4 info = make_uint4(0u, 0u, 0u, 0u);
    if (gl == 0) {
      info = __ldcg(reinterpret_cast<const uint4*>(a.lrow_info + d.w));
      __threadfence();                                 // release: the partial vectors are visible before the count
      info.w = atomicAdd(&a.lrow_info[d.w].w, 1u);
    }
    info.x = __shfl_sync(gmask, info.x, gleader); info.y = __shfl_sync(gmask, info.y, gleader);
    info.z = __shfl_sync(gmask, info.z, gleader); info.w = __shfl_sync(gmask, info.w, gleader);
    const uint32_t chunks = (info.y + kChunkRuns - 1) / kChunkRuns;
    if (info.w != chunks - 1u) continue;               // not the last chunk of the row to finish
    const uint32_t nparts = parts_of(info.y);
    if (nparts > (uint32_t)kWarpChainMax) {            // many partials: left to the whole CTA, after its last item
      uint32_t slot = 0;
      if (gl == 0) slot = atomicAdd(&s_nlong, 1u);
      slot = __shfl_sync(gmask, slot, gleader);
      if (slot < (uint32_t)kLongCap) { if (gl == 0) s_long[slot] = d.w; continue; }
    }
    __threadfence();                                   // acquire: the other chunks' partials
    finish_row<FUSED>(a, info.x, j4, chain_ring(a.partial + (int64_t)info.z * a.D + j4 * 4, nparts, a.D, mine));
  }
  finish_long_rows<FUSED>(a, stage, s_long, &s_nlong);
}

// Any row width (D a multiple of 4): one thread per (item, 16-byte lane), run after run with all copies of a run in
// flight.  Long rows only leave their partial vectors here; srm2_segment_final_kernel adds them up.
template <bool FUSED, bool PEER>
__global__ void __launch_bounds__(kRunThreads)
srm2_segment_runsum_kernel(ReduceArgs a) {
  extern __shared__ __align__(128) float4 stage[];                 // [kRunStageVecs][kRunThreads]
  float4* mine = stage + threadIdx.x;
  if (PEER && a.err != nullptr && *reinterpret_cast<const volatile uint32_t*>(a.err) != 0u) return;
  const AdamSc sc = a.sc;
  const AdamFast fa = adam_fast_prepare(sc);
  const int64_t n_lchunks = a.counters->n_lchunks;
  const int64_t items = (n_lchunks + load_nu(a.nu_host, a.nu_dev, a.cap)) * a.lpr;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int64_t t = (int64_t)blockIdx.x * kRunThreads + threadIdx.x; t < items; t += (int64_t)gridDim.x * kRunThreads) {
    int64_t c; int j4;
    if (a.shift >= 0) { c = t >> a.shift; j4 = (int)(t & (a.lpr - 1)); } else { c = t / a.lpr; j4 = (int)(t - c * a.lpr); }
    const uint4 d = c < n_lchunks ? __ldg(a.chunk_desc + c) : __ldg(a.row_desc + (c - n_lchunks));
    const int L = (int)(d.y & 0xffu);
    if (L == 0) continue;
    const bool is_long = (d.y & kLongBit) != 0, is_first = (d.y & kFirstBit) != 0;
    float* b = nullptr;
    if (!is_long) {
      const int64_t target = (int64_t)((uint64_t)d.z | ((uint64_t)d.w << 32));
      if (FUSED) {
        b = a.pool + target * (3 * (int64_t)a.D) + j4 * 4;
        cp_async16(mine + kRun * kRunThreads, b); cp_async16(mine + (kRun + 1) * kRunThreads, b + a.D);
        cp_async16(mine + (kRun + 2) * kRunThreads, b + 2 * a.D);
      } else {
        b = a.out + target * (int64_t)a.D + j4 * 4;
      }
    }
    float4 total = zero;
    const int nruns = (L + kRun - 1) / kRun;
    for (int r = 0; r < nruns; ++r) {
      const int len_r = min(kRun, L - r * kRun);
#pragma unroll
      for (int q = 0; q < kRun; ++q)
        if (q < len_r) {
          const uint32_t pos = d.y == 1u ? d.x : __ldg(a.pos_sorted + d.x + r * kRun + q);
          stage_lookup<PEER>(a, mine + q * kRunThreads, pos, j4);
        }
      cp_async_commit();
      cp_async_wait<0>();
      float4 acc = zero;
#pragma unroll
      for (int q = 0; q < kRun; ++q)
        if (q < len_r) acc = add4(acc, mine[q * kRunThreads]);
      if (is_long && !is_first) *reinterpret_cast<float4*>(a.partial + (int64_t)(d.z + r) * a.D + j4 * 4) = acc;
      else total = add4(total, acc);
    }
    if (is_long) {
      if (is_first) *reinterpret_cast<float4*>(a.partial + (int64_t)d.z * a.D + j4 * 4) = total;
      continue;
    }
    if (FUSED) {
      float4 w = mine[kRun * kRunThreads], m = mine[(kRun + 1) * kRunThreads], v = mine[(kRun + 2) * kRunThreads];
      adam_vec4_fast(w, m, v, total, fa);
      *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
    } else {
      *reinterpret_cast<float4*>(b) = total;
    }
  }
}

// ------------------------------------------------------------------------------------------ long rows (any width)
constexpr int kFinalWarps = 4;
constexpr int kFinalThreads = kFinalWarps * 32;
constexpr int kMaxColsPerLane = 4;                 // D <= 512
constexpr int kFinalSmemBytes = 64 * 1024;         // staging buffer of one CTA

// Adds `cnt` staged partial vectors (rows of lpr float4 in shared memory) to the running totals of this lane's columns.
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

// Long rows after srm2_segment_runsum_kernel: partial vectors added in order from +0.  A CTA takes four rows at a time.
//  - a row with at most `short_rows` partials is handled by one warp: each lane copies its own 16-byte columns of all
//    partials into shared memory with cp.async in one go (every load in flight at once) and adds them up;
//  - longer rows are then handled by the whole CTA, one after another: all threads copy a chunk of `chunk_rows` partials
//    as one linear block, then warp 0 adds the chunk.
template <bool FUSED>
__global__ void __launch_bounds__(kFinalThreads)
srm2_segment_final_kernel(ReduceArgs a, int short_rows, int chunk_rows) {
  extern __shared__ __align__(128) float4 smf[];                  // kFinalSmemBytes
  __shared__ uint32_t s_j[kFinalWarps], s_nr[kFinalWarps], s_pb[kFinalWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float4* mine = smf + (size_t)warp * short_rows * a.lpr;
  if (a.err != nullptr && *reinterpret_cast<const volatile uint32_t*>(a.err) != 0u) return;   // read once per thread, before any barrier:
  const uint32_t n_lrows = a.counters->n_lrows;                                                // the run-sum kernel has ended by now
  for (uint32_t g = blockIdx.x; g * kFinalWarps < n_lrows; g += gridDim.x) {
    const uint32_t mi = g * kFinalWarps + warp;
    uint32_t j = 0, nr = 0, pb = 0;
    if (mi < n_lrows) { const uint4 info = a.lrow_info[mi]; j = info.x; nr = parts_of(info.y); pb = info.z; }
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
  uint32_t *keyA, *valA, *keyB, *valB, *hist, *dtot, *seg_start, *seg_end;
  uint4* chunk_desc; uint4* row_desc; uint32_t* names; uint4* lrow_info; SegCounters* counters; float* partial;
  int tiles, bits, passes; char* zero; size_t zero_bytes;
};

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int ceil_log2(int64_t x) { int b = 0; while (((int64_t)1 << b) < x) ++b; return b; }

static size_t seg_layout(int64_t n, int64_t cap, int64_t D, char* base, SegScratch* s) {
  const int tiles = sort_tiles(n > 0 ? n : 1);
  const int keybits = ceil_log2(cap + 1 < 2 ? 2 : cap + 1);     // keys 0..cap (cap = invalid index)
  const int passes = (keybits + kMaxRadixBits - 1) / kMaxRadixBits;
  const int bits = (keybits + passes - 1) / passes;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t nn = (size_t)(n > 0 ? n : 1), cc = (size_t)(cap + 1);
  const size_t o_ka = take(nn * 4), o_va = take((nn + 16) * 4), o_kb = take(nn * 4), o_vb = take((nn + 16) * 4);
  const size_t o_h = take(sort_hist_words(tiles, bits) * 4);
  // one zero-filled region per call: counters | digit totals | seg_start | seg_end
  const size_t zero_bytes = 256 + align_up(sort_dtot_words(tiles, bits, passes) * 4, 256) + cc * 4 * 2;
  const size_t o_z = take(zero_bytes);
  const size_t o_ct = o_z, o_dt = o_z + 256, o_ss = o_dt + align_up(sort_dtot_words(tiles, bits, passes) * 4, 256);
  // long rows have more than kChunk lookups: at most n / (kChunk + 1) of them, with at most n / kChunk + that many chunks
  const size_t max_lrows = nn / (kChunk + 1) + 2;
  const size_t o_cd = take((nn / kChunk + max_lrows) * 16), o_rd = take(cc * 16), o_nm = take((nn + 16) * 4), o_li = take(max_lrows * 16);
  const size_t max_partial = (size_t)(n / kRun) + max_lrows;     // one per run of a long row at most, and one more per long row
  const size_t o_p = take(max_partial * (size_t)D * 4);
  if (s) {
    auto u = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    s->keyA = u(o_ka); s->valA = u(o_va); s->keyB = u(o_kb); s->valB = u(o_vb); s->hist = u(o_h); s->dtot = u(o_dt);
    s->seg_start = u(o_ss); s->seg_end = u(o_ss) + cc;
    s->chunk_desc = reinterpret_cast<uint4*>(base + o_cd); s->row_desc = reinterpret_cast<uint4*>(base + o_rd); s->names = u(o_nm); s->lrow_info = reinterpret_cast<uint4*>(base + o_li);
    s->counters = reinterpret_cast<SegCounters*>(base + o_ct);
    s->partial = reinterpret_cast<float*>(base + o_p);
    s->tiles = tiles; s->bits = bits; s->passes = passes; s->zero = base + o_z; s->zero_bytes = zero_bytes;
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
    if (note_cuda(cudaFuncSetAttribute(srm2_segment_runsum_kernel<FUSED, PEER>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRunSmemBytes))) return SRM2_ERR_CUDA;
    srm2_segment_runsum_kernel<FUSED, PEER><<<grid, kRunThreads, kRunSmemBytes, st>>>(a);
  }
  return SRM2_OK;
}

// pull mode (fused, runs order only); peer_out / err: optional (sums prepared at the source, status word of the exchange)
struct PullSource { const float* const* peer_grad; int world; const uint32_t* src_code; const float* const* peer_out; const uint32_t* err; };

// phase bits: kSortPhase (radix passes) and kDescrPhase (boundaries, plan, item descriptors) together are the index half —
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
  // lookup positions and sorted indices are 32-bit
  if ((D & 3) != 0 || D > 128 * kMaxColsPerLane || n >= ((int64_t)1 << 31) - 64 || cap >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (sum_phase && ((n > 0 && !pull && !aligned16(grad)) || (fused ? !aligned16(pool) : !aligned16(out)))) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < seg_layout(n, cap, D, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  SegScratch s;
  seg_layout(n, cap, D, static_cast<char*>(scratch), &s);
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  const bool small = order == SRM2_ORDER_WINDOWS || (order == SRM2_ORDER_AUTO && n <= kSmallN);
  const bool wide = (lpr == 16 || lpr == 32);            // an item's lanes are an aligned half or whole warp of >= kRun lanes
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
    srm2_segment_bounds_kernel<<<index_grid((n + 255) / 256), 256, 0, st>>>(skey, spos, n, n_dev, s.seg_start, s.seg_end, cap,
                                                                           pull ? pull->src_code : nullptr, s.names);
    ++launches;
  }
  ReduceArgs a{};
  a.grad = grad; a.D = (int)D; a.lpr = lpr; a.shift = shift; a.skey = skey; a.spos = spos; a.seg_start = s.seg_start; a.seg_end = s.seg_end;
  // what names a lookup's gradient row: its position (the sort's value array), or in pull mode its (rank, row) code
  a.chunk_desc = s.chunk_desc; a.row_desc = s.row_desc; a.pos_sorted = pull ? s.names : spos; a.lrow_info = s.lrow_info; a.counters = s.counters;
  a.inplace = wide ? 1 : 0; a.partial = s.partial;
  a.out = out; a.pool = pool; a.slots = slots;
  if (fused && sum_phase) a.sc = AdamSc{sc[0], sc[1], sc[2], sc[3], sc[4], sc[5], sc[6], sc[7]};
  a.nu_host = nu_host; a.nu_dev = nu_dev; a.cap = cap; a.n = n;
  if (pull && sum_phase) {
    for (int r = 0; r < pull->world; ++r) {
      a.peer[r] = pull->peer_grad[r];
      a.peer_out[r] = pull->peer_out ? pull->peer_out[r] : nullptr;
    }
    a.err = pull->err;
  }
  if (small) {
    const int64_t row_items = cap * lpr;
    const int grid_rows = (int)((row_items + 255) / 256 < (int64_t)kSMs * 16 ? (row_items + 255) / 256 : (int64_t)kSMs * 16);
    stage_begin(st);
    if (fused) srm2_segment_windowed_kernel<true><<<grid_rows, 256, 0, st>>>(a);
    else srm2_segment_windowed_kernel<false><<<grid_rows, 256, 0, st>>>(a);
    stage_end(st);
    return launch_status(launches + 1);
  }
  // 3. plan.  A split call leaves rows without lookups alone (its index half must not write rows).
  if (sort_phase && !descr_phase && !sum_phase) return launch_status(launches);
  if (descr_phase) {
    const int skip_empty = phase != kAllPhases;
    const unsigned plan_blocks = index_grid((cap + kPlanThreads - 1) / kPlanThreads);
    if (fused) srm2_segment_plan_kernel<true><<<plan_blocks, kPlanThreads, 0, st>>>(a, s.chunk_desc, s.row_desc, s.counters, skip_empty);
    else srm2_segment_plan_kernel<false><<<plan_blocks, kPlanThreads, 0, st>>>(a, s.chunk_desc, s.row_desc, s.counters, skip_empty);
    launches += 1;
    if (!sum_phase) return launch_status(launches);
  }
  // 4. run sums (and, for widths whose lane groups do not sit inside a warp, a second kernel for the long rows)
  const int64_t run_items_max = (n / kChunk + n / (kChunk + 1) + 2 + cap) * lpr;      // long chunks + one entry per unique row
  // Many short-lived CTAs: a CTA that has to add up a row of many partial vectors does so after its last item, so the
  // sooner CTAs end the sooner those chains start; in the split form SM room also frees up every few microseconds for the
  // small kernels of the other streams (the next steps' index work).  CTAs of 128 threads, eight to an SM, 64 per SM in all:
  // the eight hold every register of the SM between them, so the finer the grain the sooner another kernel's CTA gets in.
  const int64_t cta_cap = (int64_t)kSMs * 64;
  const int grid_runs = (int)((run_items_max + kRunThreads - 1) / kRunThreads < cta_cap ? (run_items_max + kRunThreads - 1) / kRunThreads : cta_cap);
  const int rows_fit = (int)(kFinalSmemBytes / (D * 4));                 // partial vectors that fit the CTA's staging buffer
  const int short_rows = rows_fit / kFinalWarps, chunk_rows = rows_fit;
  const size_t sm_final = kFinalSmemBytes;
  const int64_t groups_max = (n / (kChunk + 1) + kFinalWarps) / kFinalWarps;
  const int grid_final = (int)(groups_max < (int64_t)kSMs * 3 ? groups_max : (int64_t)kSMs * 3);
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
  const srm2::PullSource pull{peer_grad, (int)world, src_code, nullptr, nullptr};
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, nullptr, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), &pull);
}

extern "C" int srm2_reduce_adam_index(const int64_t* slots, const uint32_t* src_code, const int64_t* inv, int64_t n, const int64_t* n_dev,
                                      int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, int part, void* scratch,
                                      size_t scratch_bytes, srm2_stream_t stream) {
  if (part < 0 || part > 2) return SRM2_ERR_ARG;
  const srm2::PullSource pull{nullptr, 1, src_code, nullptr, nullptr};
  const int phase = part == SRM2_INDEX_SORT ? srm2::kSortPhase : (part == SRM2_INDEX_DESCRIPTORS ? srm2::kDescrPhase : srm2::kIndexPhase);
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, nullptr, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, nullptr, slots, nullptr,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), src_code ? &pull : nullptr, phase);
}

extern "C" int srm2_reduce_adam_apply_f32(float* pool, const int64_t* slots, const float* grad, const float* const* peer_grad, int64_t world,
                                          int64_t n, const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev,
                                          int64_t max_unique, const float sc[8], void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  if ((grad == nullptr) == (peer_grad == nullptr) && n > 0) return SRM2_ERR_ARG;       // exactly one gradient source
  if (peer_grad != nullptr && (world < 1 || world > srm2::kMaxGradPeers)) return SRM2_ERR_ARG;
  const srm2::PullSource pull{peer_grad, (int)world, nullptr, nullptr, nullptr};
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, grad, nullptr, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), peer_grad ? &pull : nullptr, srm2::kSumPhase);
}

extern "C" int srm2_reduce_adam_apply_pull_f32(float* pool, const int64_t* slots, const float* const* peer_grad, const float* const* peer_out,
                                               const uint32_t* err, int64_t world, int64_t n, const int64_t* n_dev, int64_t D, int64_t n_unique,
                                               const int64_t* n_unique_dev, int64_t max_unique, const float sc[8], void* scratch,
                                               size_t scratch_bytes, srm2_stream_t stream) {
  if (peer_grad == nullptr || world < 1 || world > srm2::kMaxGradPeers) return SRM2_ERR_ARG;
  for (int r = 0; peer_out != nullptr && r < world; ++r)
    if (peer_out[r] == nullptr || !srm2::aligned16(peer_out[r])) return SRM2_ERR_ARG;
  const srm2::PullSource pull{peer_grad, (int)world, nullptr, peer_out, err};
  return srm2::segment_pipeline(true, SRM2_ORDER_RUNS, nullptr, nullptr, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream), &pull, srm2::kSumPhase);
}

// ------------------------------------------------------------------------------------------ sums prepared at the source
// Owner side.  After the descriptors of a step: one thread per run of every row looks at the run's leading lookups that
// come from one other rank; two or more of them are replaced by a single row that the source rank will have summed (in
// the same order, from +0) and stored into this rank's buffer of sums by the time the run-sum kernel reads it.  The thread
// takes the next free request entry for that source (atomic counters; which entry a run gets does not matter), stores
// the request into the source's request buffer over NVLink, and renames the run's lookups: the first one to the entry in
// this rank's buffer of sums (region of that source), the others to kSkipName.  A run that finds the request buffer full
// stays as it is: its rows are then read from the source one by one, as without any of this.  Every other lookup of
// another rank — further back in a run, or alone at its head — becomes a request for a single row, so that it, too,
// arrives in this rank's memory instead of being read over NVLink by the run-sum kernel.
namespace srm2 {

__global__ void __launch_bounds__(256)
srm2_presum_request_kernel(const uint32_t* __restrict__ skey, const uint32_t* __restrict__ seg_start, const uint32_t* __restrict__ seg_end,
                           uint32_t* __restrict__ names, uint4* __restrict__ row_desc, int64_t n_host, const int64_t* __restrict__ n_dev,
                           int64_t cap_rows, int rank, int world, uint32_t cap_req, PeerPtrs req, uint32_t* __restrict__ req_count, PeerPtrs req_n,
                           PeerPtrs sig, unsigned long long ticket, uint32_t* __restrict__ err, long long timeout_ns) {
  __shared__ uint32_t s_cnt[kMaxPeers], s_base[kMaxPeers];
  __shared__ bool s_last;
  const int64_t n = eff_count(n_host, n_dev);
  const int64_t n_round = (n + 255) / 256 * 256;
  const uint32_t pm = kOutBit - 1u;
  bool wrote = false;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n_round; i += (int64_t)gridDim.x * 256) {
    if (threadIdx.x < kMaxPeers) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    // the thread at the head of a run looks after the whole run
    uint32_t nm[kRun], k = 0;
    int m_max = 0, m = 0;
    bool lone = false;
    if (i < n) {
      k = skey[i];
      if ((int64_t)k < cap_rows) {
        const uint32_t s = seg_start[k], e = seg_end[k];
        if (((uint32_t)i - s) % (uint32_t)kRun == 0u) { m_max = (int)min((uint32_t)kRun, e - (uint32_t)i); lone = e - s == 1u; }
      }
    }
#pragma unroll
    for (int q = 0; q < kRun; ++q) nm[q] = q < m_max ? names[i + q] : kSkipName;
    auto from_peer = [&](uint32_t code) { const uint32_t r = code >> kPeerShift; return r != (uint32_t)rank && r < (uint32_t)world; };
    if (m_max > 0 && from_peer(nm[0])) {               // the leading lookups that come from the rank of the first one
      m = 1;
      bool same = true;
#pragma unroll
      for (int q = 1; q < kRun; ++q) { same = same && (nm[q] >> kPeerShift) == (nm[0] >> kPeerShift); m += same ? 1 : 0; }
    }
    // one request for the leading group (m rows), one for every later lookup of another rank; first a place among the CTA's
    // requests for the same source, then one range per source and CTA, taken from the source's counter
    uint32_t loc[kRun];
    uint32_t asks = 0;
#pragma unroll
    for (int q = 0; q < kRun; ++q) {
      const bool a = q < m_max && (q == 0 ? m >= 1 : (q >= m && from_peer(nm[q])));
      if (a) { asks |= 1u << q; loc[q] = atomicAdd(s_cnt + (nm[q] >> kPeerShift), 1u); }
    }
    __syncthreads();
    if ((int)threadIdx.x < world && s_cnt[threadIdx.x] != 0u) s_base[threadIdx.x] = atomicAdd(req_count + threadIdx.x, s_cnt[threadIdx.x]);
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kRun; ++q) {
      if (!(asks >> q & 1u)) continue;
      const uint32_t src = nm[q] >> kPeerShift, idx = s_base[src] + loc[q];
      if (idx >= cap_req) continue;                    // no room in the source's buffer: these lookups stay as they are
      uint4* r = static_cast<uint4*>(req.p[src]) + ((size_t)rank * cap_req + idx) * (kReqWords / 4);
      if (q == 0 && m >= 2) {
        r[0] = make_uint4((uint32_t)m, nm[0] & pm, nm[1] & pm, m > 2 ? nm[2] & pm : 0u);
        r[1] = make_uint4(m > 3 ? nm[3] & pm : 0u, m > 4 ? nm[4] & pm : 0u, m > 5 ? nm[5] & pm : 0u, m > 6 ? nm[6] & pm : 0u);
        r[2] = make_uint4(m > 7 ? nm[7] & pm : 0u, m > 8 ? nm[8] & pm : 0u, m > 9 ? nm[9] & pm : 0u, 0u);
#pragma unroll
        for (int e = 1; e < kRun; ++e)
          if (e < m) names[i + e] = kSkipName;
      } else {
        r[0] = make_uint4(1u, nm[q] & pm, 0u, 0u); r[1] = make_uint4(0u, 0u, 0u, 0u); r[2] = make_uint4(0u, 0u, 0u, 0u);
      }
      const uint32_t renamed = (src << kPeerShift) | kOutBit | idx;
      names[i + q] = renamed;
      if (lone) row_desc[k].x = renamed;               // a row of one lookup carries the name in its descriptor
      wrote = true;
    }
    __syncthreads();                                   // s_cnt and s_base are reused by the next round
  }
  // the last CTA to finish tells every source how many requests this rank has left in its buffer, leaves the counters
  // zero for the next call, and goes through the barrier: all ranks have left their requests everywhere
  if (wrote) __threadfence_system();
  __syncthreads();
  uint32_t* done = req_count + kMaxPeers;
  if (threadIdx.x == 0) { __threadfence(); s_last = atomicAdd(done, 1u) == gridDim.x - 1u; }
  __syncthreads();
  if (!s_last) return;
  const int sidx = threadIdx.x;
  if (sidx < world) {
    const uint32_t c = min(*reinterpret_cast<volatile uint32_t*>(req_count + sidx), cap_req);
    static_cast<uint32_t*>(req_n.p[sidx])[rank] = c;
    req_count[sidx] = 0u;
    __threadfence_system();
  }
  if (sidx == 0) *done = 0u;
  if (sidx < 32) __syncwarp();
  if (sidx < world && ticket != 0) peer_barrier_lane(sig, rank, sidx, ticket, err, timeout_ns);
}

}  // namespace srm2

extern "C" int srm2_presum_request(int64_t n, const int64_t* n_dev, int64_t D, int64_t max_unique, void* scratch, size_t scratch_bytes,
                                   const srm2_presum* ps, srm2_stream_t stream) {
  using namespace srm2;
  if (ps == nullptr || n < 0 || D <= 0 || max_unique < 0) return SRM2_ERR_ARG;
  const int64_t W = ps->world;
  if (W < 1 || W > kMaxPeers || ps->rank < 0 || ps->rank >= W || ps->cap < 1 || ps->cap >= (int64_t)kOutBit || ps->peer_req == nullptr ||
      ps->peer_req_n == nullptr || ps->req_count == nullptr || ps->err == nullptr)
    return SRM2_ERR_ARG;
  if (ps->ticket != 0 && (ps->peer_tickets == nullptr || ps->timeout_ns <= 0)) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || n >= (int64_t)kOutBit || max_unique >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;   // positions must leave kOutBit free
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < seg_layout(n, max_unique, D, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  PeerPtrs pr{}, pn{}, pt{};
  for (int r = 0; r < W; ++r) {
    if (ps->peer_req[r] == nullptr || !aligned16(ps->peer_req[r]) || ps->peer_req_n[r] == nullptr) return SRM2_ERR_ARG;
    if (ps->ticket != 0 && ps->peer_tickets[r] == nullptr) return SRM2_ERR_ARG;
    pr.p[r] = ps->peer_req[r]; pn.p[r] = ps->peer_req_n[r]; pt.p[r] = ps->ticket != 0 ? ps->peer_tickets[r] : nullptr;
  }
  SegScratch s;
  seg_layout(n, max_unique, D, static_cast<char*>(scratch), &s);
  const uint32_t* skey = (s.passes & 1) ? s.keyA : s.keyB;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t req_blocks = (n + 255) / 256 < (int64_t)kSMs ? (n + 255) / 256 : (int64_t)kSMs;      // one CTA per SM: see index_grid
  srm2_presum_request_kernel<<<(unsigned)(req_blocks < 1 ? 1 : req_blocks), 256, 0, st>>>(skey, s.seg_start, s.seg_end, s.names, s.row_desc, n, n_dev, max_unique,
                                                                        (int)ps->rank, (int)W, (uint32_t)ps->cap, pr, ps->req_count, pn, pt,
                                                                        (unsigned long long)ps->ticket, ps->err, (long long)ps->timeout_ns);
  return launch_status(1);
}

extern "C" int srm2_reduce_adam_nd_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n,
                                       const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev,
                                       int64_t max_unique, int order, const float sc[8], void* scratch, size_t scratch_bytes,
                                       srm2_stream_t stream) {
  return srm2::segment_pipeline(true, order, grad, inv, n, n_dev, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}
