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
//   1. stable LSD radix sort of (key = inverse index, value = lookup position), 32-bit keys, up to 11 bits per pass;
//      the number of passes follows from the bound on the number of unique rows, so typical inputs take two.
//   2. segment starts from the sorted keys; per-segment run counts; exclusive scans of those (single CTA).
//   3. run descriptors; one thread group per run sums its <= 10 gradient rows (all loads issued up front) — work is
//      balanced over the whole GPU however long the longest segment is; rows with a single run are finished here.
//   4. rows with several runs: run sums added in order (partials are L2 resident), then written / Adam applied.
// Gradient rows are read exactly once (D*4 bytes per lookup); everything else is small integer traffic.
#include "common.cuh"
#include "scan.cuh"
#include "sort.cuh"

namespace srm2 {

constexpr int kRun = 10;            // lookups per run (large inputs)
constexpr int kSmallN = 3072;       // inputs up to this many lookups use the windowed order
constexpr int kWindow = 32;

// ------------------------------------------------------------------------------------------ segments
// seg_start[j] = number of sorted keys below j (lower bound), for j in [0, nu]; a row without lookups gets an empty
// segment.  Keys are clamped to `cap` by the sort, so lookups with an invalid index land behind every segment.
__global__ void __launch_bounds__(256)
srm2_segment_bounds_kernel(const uint32_t* __restrict__ skey, int64_t n, uint32_t* __restrict__ seg_start,
                           int64_t nu_host, const int64_t* __restrict__ nu_dev, int64_t cap) {
  int64_t nu = nu_dev ? *nu_dev : nu_host; if (nu > cap) nu = cap;
  for (int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x; j <= nu; j += (int64_t)gridDim.x * 256) {
    int64_t lo = 0, hi = n;
    while (lo < hi) { const int64_t mid = (lo + hi) >> 1; if ((int64_t)skey[mid] < j) lo = mid + 1; else hi = mid; }
    seg_start[j] = (uint32_t)lo;
  }
}

// runs[j] = number of runs of segment j; mruns[j] = the same if the segment has more than one run, else 0.
__global__ void __launch_bounds__(256)
srm2_segment_runs_kernel(const uint32_t* __restrict__ seg_start, uint32_t* __restrict__ runs, uint32_t* __restrict__ mruns,
                         int64_t nu_host, const int64_t* __restrict__ nu_dev, int64_t cap) {
  int64_t nu = nu_dev ? *nu_dev : nu_host; if (nu > cap) nu = cap;
  for (int64_t j = (int64_t)blockIdx.x * 256 + threadIdx.x; j < nu; j += (int64_t)gridDim.x * 256) {
    const uint32_t len = seg_start[j + 1] - seg_start[j];
    const uint32_t r = (len + kRun - 1) / kRun;
    runs[j] = r; mruns[j] = r > 1 ? r : 0u;
  }
}

// run_first[c] = sorted index of the first lookup of run c.
__global__ void __launch_bounds__(256)
srm2_segment_descr_kernel(const uint32_t* __restrict__ skey, int64_t n, const uint32_t* __restrict__ seg_start,
                          const uint32_t* __restrict__ run_base, uint32_t* __restrict__ run_first, int64_t nu_host,
                          const int64_t* __restrict__ nu_dev, int64_t cap) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  int64_t nu = nu_dev ? *nu_dev : nu_host; if (nu > cap) nu = cap;
  const uint32_t j = skey[i];
  if ((int64_t)j >= nu) return;
  const uint32_t off = (uint32_t)i - seg_start[j];
  if (off % kRun == 0) run_first[run_base[j] + off / kRun] = (uint32_t)i;
}

struct ReduceArgs {
  const float* grad; int D; int lpr; int shift;
  const uint32_t* skey; const uint32_t* spos; const uint32_t* seg_start;
  const uint32_t* run_base; const uint32_t* mrun_base; const uint32_t* run_first; const uint32_t* n_runs;
  float* partial;
  float* out;               // [nu, D] (unfused) or nullptr
  float* pool; const int64_t* slots; AdamSc sc;   // fused Adam: pool [C,3,D], slots[j] = pool row of unique row j
  int64_t nu_host; const int64_t* nu_dev; int64_t cap; int64_t n;
};

__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// Writes the finished gradient sum of unique row j (lane j4): either into out, or through Adam into the pool.
template <bool FUSED>
__device__ __forceinline__ void finish_row(const ReduceArgs& a, uint32_t j, int j4, const float4& g) {
  if (FUSED) {
    float* b = a.pool + a.slots[j] * (3 * (int64_t)a.D) + j4 * 4;
    float4 w = *reinterpret_cast<const float4*>(b), m = *reinterpret_cast<const float4*>(b + a.D),
           v = *reinterpret_cast<const float4*>(b + 2 * a.D);
    adam_vec4(w, m, v, g, a.sc);
    *reinterpret_cast<float4*>(b) = w; *reinterpret_cast<float4*>(b + a.D) = m; *reinterpret_cast<float4*>(b + 2 * a.D) = v;
  } else {
    *reinterpret_cast<float4*>(a.out + (int64_t)j * a.D + j4 * 4) = g;
  }
}

// One thread per (run, 16-byte lane).  Sums the <= 10 gradient rows of the run from +0; a row with a single run is
// finished here ((+0) + run sum), otherwise the run sum goes to the partial buffer.
template <bool FUSED>
__global__ void __launch_bounds__(256)
srm2_segment_runsum_kernel(ReduceArgs a) {
  const int64_t items = (int64_t)(*a.n_runs) * a.lpr;
  for (int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x; t < items; t += (int64_t)gridDim.x * 256) {
    int64_t c; int j4;
    if (a.shift >= 0) { c = t >> a.shift; j4 = (int)(t & (a.lpr - 1)); } else { c = t / a.lpr; j4 = (int)(t - c * a.lpr); }
    const uint32_t first = a.run_first[c];
    const uint32_t j = a.skey[first];
    const uint32_t s0 = a.seg_start[j], s1 = a.seg_start[j + 1];
    const uint32_t len = min((uint32_t)kRun, s1 - first);
    float4 g[kRun];
#pragma unroll
    for (int q = 0; q < kRun; ++q)
      if (q < (int)len) g[q] = ld_stream4(a.grad + (int64_t)a.spos[first + q] * a.D + j4 * 4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kRun; ++q)
      if (q < (int)len) acc = add4(acc, g[q]);
    if (s1 - s0 <= (uint32_t)kRun) {
      finish_row<FUSED>(a, j, j4, add4(make_float4(0.f, 0.f, 0.f, 0.f), acc));
    } else {
      const uint32_t slot = a.mrun_base[j] + (first - s0) / kRun;
      *reinterpret_cast<float4*>(a.partial + (int64_t)slot * a.D + j4 * 4) = acc;
    }
  }
}

// One thread per (unique row, lane): rows with several runs add their run sums in order, from +0.
template <bool FUSED>
__global__ void __launch_bounds__(256)
srm2_segment_final_kernel(ReduceArgs a) {
  int64_t nu = a.nu_dev ? *a.nu_dev : a.nu_host; if (nu > a.cap) nu = a.cap;
  const int64_t items = nu * a.lpr;
  for (int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x; t < items; t += (int64_t)gridDim.x * 256) {
    int64_t j; int j4;
    if (a.shift >= 0) { j = t >> a.shift; j4 = (int)(t & (a.lpr - 1)); } else { j = t / a.lpr; j4 = (int)(t - j * a.lpr); }
    const uint32_t len = a.seg_start[j + 1] - a.seg_start[j];
    if (len == 0) { finish_row<FUSED>(a, (uint32_t)j, j4, make_float4(0.f, 0.f, 0.f, 0.f)); continue; }   // no lookups: zero gradient
    if (len <= (uint32_t)kRun) continue;
    const uint32_t nr = (len + kRun - 1) / kRun;
    const float* p = a.partial + (int64_t)a.mrun_base[j] * a.D + j4 * 4;
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
    uint32_t c = 0;
    for (; c + 8 <= nr; c += 8) {
      float4 x[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) x[q] = *reinterpret_cast<const float4*>(p + (int64_t)(c + q) * a.D);
#pragma unroll
      for (int q = 0; q < 8; ++q) tot = add4(tot, x[q]);
    }
    for (; c < nr; ++c) tot = add4(tot, *reinterpret_cast<const float4*>(p + (int64_t)c * a.D));
    finish_row<FUSED>(a, (uint32_t)j, j4, tot);
  }
}

// Small inputs: one thread per (unique row, lane) walks the row's lookups in ascending position; lookups of the same
// 32-position window are summed from the first one, each window sum is then added to the row total (from +0).
template <bool FUSED>
__global__ void __launch_bounds__(256)
srm2_segment_windowed_kernel(ReduceArgs a) {
  int64_t nu = a.nu_dev ? *a.nu_dev : a.nu_host; if (nu > a.cap) nu = a.cap;
  const int64_t items = nu * a.lpr;
  for (int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x; t < items; t += (int64_t)gridDim.x * 256) {
    int64_t j; int j4;
    if (a.shift >= 0) { j = t >> a.shift; j4 = (int)(t & (a.lpr - 1)); } else { j = t / a.lpr; j4 = (int)(t - j * a.lpr); }
    const uint32_t s0 = a.seg_start[j], s1 = a.seg_start[j + 1];
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
  uint32_t *keyA, *valA, *keyB, *valB, *hist, *seg_start, *runs, *mruns, *run_first, *n_runs;
  float* partial;
  int tiles, bits, passes;
};

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int ceil_log2(int64_t x) { int b = 0; while (((int64_t)1 << b) < x) ++b; return b; }

static size_t seg_layout(int64_t n, int64_t cap, int64_t D, char* base, SegScratch* s) {
  const int tiles = (int)((n + kSortTile - 1) / kSortTile);
  const int keybits = ceil_log2(cap + 1 < 2 ? 2 : cap + 1);     // keys 0..cap (cap = invalid index)
  const int passes = (keybits + kMaxRadixBits - 1) / kMaxRadixBits;
  const int bits = (keybits + passes - 1) / passes;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t nn = (size_t)(n > 0 ? n : 1);
  const size_t o_ka = take(nn * 4), o_va = take(nn * 4), o_kb = take(nn * 4), o_vb = take(nn * 4);
  const size_t o_h = take(((size_t)tiles * ((size_t)1 << bits) + 1) * 4);
  const size_t o_ss = take((size_t)(cap + 2) * 4), o_r = take((size_t)(cap + 2) * 4), o_mr = take((size_t)(cap + 2) * 4);
  const size_t o_rf = take(nn * 4), o_nr = take(16);
  const size_t max_partial = (size_t)(n / kRun + n / (kRun + 1) + 2);
  const size_t o_p = take(max_partial * (size_t)D * 4);
  if (s) {
    auto u = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    s->keyA = u(o_ka); s->valA = u(o_va); s->keyB = u(o_kb); s->valB = u(o_vb); s->hist = u(o_h); s->seg_start = u(o_ss);
    s->runs = u(o_r); s->mruns = u(o_mr); s->run_first = u(o_rf); s->n_runs = u(o_nr);
    s->partial = reinterpret_cast<float*>(base + o_p);
    s->tiles = tiles; s->bits = bits; s->passes = passes;
  }
  return off;
}

static int segment_pipeline(bool fused, int order, const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t nu_host,
                            const int64_t* nu_dev, int64_t cap, float* out, float* pool, const int64_t* slots,
                            const float* sc, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (n < 0 || D <= 0 || cap < 0 || (nu_host < 0 && nu_dev == nullptr) || order < 0 || order > 2) return SRM2_ERR_ARG;
  if (nu_dev == nullptr) cap = nu_host;
  if (cap == 0) return SRM2_OK;
  if (n > 0 && (grad == nullptr || inv == nullptr)) return SRM2_ERR_ARG;
  if (fused ? (pool == nullptr || slots == nullptr || sc == nullptr) : out == nullptr) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || D > (1 << 16) || n >= ((int64_t)1 << 31) || cap >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (!aligned16(grad) || (fused ? !aligned16(pool) : !aligned16(out))) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < seg_layout(n, cap, D, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  SegScratch s;
  seg_layout(n, cap, D, static_cast<char*>(scratch), &s);
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;

  // 1. sort (key = inv, value = position)
  const uint32_t *skey = nullptr, *spos = nullptr;
  if (n > 0) {
    SortBuffers sb{s.keyA, s.valA, s.keyB, s.valB, s.hist, s.tiles};
    const int rc = radix_sort_by_key(inv, n, /*mod=*/0, cap, s.bits, s.passes, sb, &skey, &spos, st);
    if (rc != SRM2_OK) return rc;
  }
  // 2. segment starts
  const int grid_n = (int)((n + 255) / 256 > 0 ? (n + 255) / 256 : 1);
  const int grid_u = (int)((cap + 256) / 256 < (int64_t)kSMs * 8 ? (cap + 256) / 256 : (int64_t)kSMs * 8);
  srm2_segment_bounds_kernel<<<grid_u, 256, 0, st>>>(skey, n, s.seg_start, nu_host, nu_dev, cap);
  ReduceArgs a{};
  a.grad = grad; a.D = (int)D; a.lpr = lpr; a.shift = shift; a.skey = skey; a.spos = spos; a.seg_start = s.seg_start;
  a.run_base = s.runs; a.mrun_base = s.mruns; a.run_first = s.run_first; a.n_runs = s.n_runs; a.partial = s.partial;
  a.out = out; a.pool = pool; a.slots = slots;
  if (fused) a.sc = AdamSc{sc[0], sc[1], sc[2], sc[3], sc[4], sc[5], sc[6], sc[7]};
  a.nu_host = nu_host; a.nu_dev = nu_dev; a.cap = cap; a.n = n;
  const int64_t row_items = cap * lpr;
  const int grid_rows = (int)((row_items + 255) / 256 < (int64_t)kSMs * 16 ? (row_items + 255) / 256 : (int64_t)kSMs * 16);
  int launches = n > 0 ? 3 * s.passes + 1 : 1;
  if (order == SRM2_ORDER_WINDOWS || (order == SRM2_ORDER_AUTO && n <= kSmallN)) {
    stage_begin(st);
    if (fused) srm2_segment_windowed_kernel<true><<<grid_rows, 256, 0, st>>>(a);
    else srm2_segment_windowed_kernel<false><<<grid_rows, 256, 0, st>>>(a);
    stage_end(st);
    return launch_status(launches + 1);
  }
  // 3. runs per segment, their exclusive scans, run descriptors
  srm2_segment_runs_kernel<<<grid_u, 256, 0, st>>>(s.seg_start, s.runs, s.mruns, nu_host, nu_dev, cap);
  srm2_scan_exclusive_u32_kernel<<<1, kScanThreads, 0, st>>>(s.runs, s.runs, nu_host, nu_dev, cap, 0, s.n_runs);
  srm2_scan_exclusive_u32_kernel<<<1, kScanThreads, 0, st>>>(s.mruns, s.mruns, nu_host, nu_dev, cap, 0, nullptr);
  srm2_segment_descr_kernel<<<grid_n, 256, 0, st>>>(skey, n, s.seg_start, s.runs, s.run_first, nu_host, nu_dev, cap);
  // 4. run sums, then multi-run rows
  const int64_t run_items_max = n * lpr;
  const int grid_runs = (int)((run_items_max + 255) / 256 < (int64_t)kSMs * 16 ? (run_items_max + 255) / 256 : (int64_t)kSMs * 16);
  stage_begin(st);
  if (fused) {
    srm2_segment_runsum_kernel<true><<<grid_runs, 256, 0, st>>>(a);
    srm2_segment_final_kernel<true><<<grid_rows, 256, 0, st>>>(a);
  } else {
    srm2_segment_runsum_kernel<false><<<grid_runs, 256, 0, st>>>(a);
    srm2_segment_final_kernel<false><<<grid_rows, 256, 0, st>>>(a);
  }
  stage_end(st);
  return launch_status(launches + 6);
}

}  // namespace srm2

extern "C" size_t srm2_segment_scratch_bytes(int64_t n, int64_t max_unique, int64_t D) {
  if (n < 0 || max_unique < 0 || D <= 0) return 0;
  return srm2::seg_layout(n, max_unique, D, nullptr, nullptr);
}

extern "C" int srm2_segment_reduce_f32(const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t n_unique,
                                       const int64_t* n_unique_dev, int64_t max_unique, int order, float* out, void* scratch,
                                       size_t scratch_bytes, srm2_stream_t stream) {
  return srm2::segment_pipeline(false, order, grad, inv, n, D, n_unique, n_unique_dev, max_unique, out, nullptr, nullptr, nullptr,
                                scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int srm2_reduce_adam_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n,
                                    int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique,
                                    int order, const float sc[8], void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  return srm2::segment_pipeline(true, order, grad, inv, n, D, n_unique, n_unique_dev, max_unique, nullptr, pool, slots, sc, scratch,
                                scratch_bytes, static_cast<cudaStream_t>(stream));
}
