// Pull exchange, source side of the prepared sums: the owners of a step's rows have left requests in this rank's request
// buffer (srm2_presum_request) — each names up to ten of this rank's gradient rows that open a run of one unique row (or
// a single row further back in a run).  The kernel adds them in the requested order, starting from +0, exactly as the
// owner's run-sum kernel would have after reading them one by one over NVLink, and stores the sum into the owner's buffer
// of sums (peer stores): one row crosses instead of up to ten, and the owner's run-sum kernel reads local memory only.
// The gradient rows are read from local memory.
#include "common.cuh"
#include "peer.cuh"

namespace srm2 {
namespace {

constexpr int kRun = 10, kPresumThreads = 256;   // a request: 12 words {m, positions[10], unused}

__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
  return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// One thread per (request, 16-byte lane).  Requests of owner o are entries [0, req_n[o]) of region o of the request
// buffer; region `rank` is unused (an owner never asks itself).  The last CTA to finish goes through the barrier: every
// rank's sums are in place before any rank's run-sum kernel starts.
__global__ void __launch_bounds__(kPresumThreads, 3)
srm2_presum_rows_kernel(const float* __restrict__ grad, int64_t n, int lpr, int shift, int D, int world, int rank, uint32_t cap_req,
                        const uint4* __restrict__ req, const uint32_t* __restrict__ req_n, PeerPtrs out, uint32_t* __restrict__ err,
                        PeerPtrs sig, unsigned long long ticket, long long timeout_ns, uint32_t* __restrict__ done) {
  __shared__ uint32_t s_pre[kMaxPeers + 1];
  __shared__ bool s_last;
  if (threadIdx.x == 0) {
    uint32_t acc = 0;
    for (int o = 0; o < world; ++o) { s_pre[o] = acc; acc += o == rank ? 0u : min(req_n[o], cap_req); }
    for (int o = world; o <= kMaxPeers; ++o) s_pre[o] = acc;
  }
  __syncthreads();
  const int64_t items = (int64_t)s_pre[world] * lpr;
  const int64_t step = (int64_t)gridDim.x * kPresumThreads;
  // the request of the thread's next item is fetched while the rows of this one are in flight
  auto entry_of = [&](int64_t t, int& j4, float*& dst) -> size_t {
    int64_t rq;
    if (shift >= 0) { rq = t >> shift; j4 = (int)(t & (lpr - 1)); } else { rq = t / lpr; j4 = (int)(t - rq * lpr); }
    int o = 0;
    while (o + 1 < world && (uint32_t)rq >= s_pre[o + 1]) ++o;
    const uint32_t idx = (uint32_t)rq - s_pre[o];
    dst = static_cast<float*>(out.p[o]) + (int64_t)idx * D + j4 * 4;        // owner o's buffer of sums, this rank's region
    return (size_t)o * cap_req + idx;
  };
  int64_t t = (int64_t)blockIdx.x * kPresumThreads + threadIdx.x;
  int j4 = 0, j4n = 0;
  size_t entry = 0, entry_n = 0;
  float *dst = nullptr, *dst_n = nullptr;
  uint4 r0 = make_uint4(0u, 0u, 0u, 0u), r1 = r0, r2 = r0;
  if (t < items) { entry = entry_of(t, j4, dst); r0 = __ldg(req + entry * 3); r1 = __ldg(req + entry * 3 + 1); r2 = __ldg(req + entry * 3 + 2); }
  for (; t < items; t += step) {
    const uint32_t pos[kRun] = {r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w, r2.x, r2.y, r2.z};
    const int m = (int)min(r0.x, (uint32_t)kRun);
    float4 v[kRun];
    bool bad = false;
#pragma unroll
    for (int q = 0; q < kRun; ++q)
      if (q < m) {
        uint32_t p = pos[q];
        if ((int64_t)p >= n) { bad = true; p = 0; }
        v[q] = __ldg(reinterpret_cast<const float4*>(grad + (int64_t)p * D + j4 * 4));
      }
    if (t + step < items) {
      entry_n = entry_of(t + step, j4n, dst_n);
      r0 = __ldg(req + entry_n * 3); r1 = __ldg(req + entry_n * 3 + 1); r2 = __ldg(req + entry_n * 3 + 2);
    }
    if (bad) atomicOr(err, 8u);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kRun; ++q)
      if (q < m) acc = add4(acc, v[q]);
    *reinterpret_cast<float4*>(dst) = acc;
    entry = entry_n; j4 = j4n; dst = dst_n;
  }
  if (ticket == 0) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x == 0) *done = 0u;                    // ready for the next launch
  if ((int)threadIdx.x < world) peer_barrier_lane(sig, rank, (int)threadIdx.x, ticket, err, timeout_ns);
}

}  // namespace
}  // namespace srm2

extern "C" int srm2_presum_rows_f32(const float* grad, int64_t n, int64_t D, const srm2_presum* ps, srm2_stream_t stream) {
  using namespace srm2;
  if (ps == nullptr || n < 0 || D <= 0) return SRM2_ERR_ARG;
  const int64_t W = ps->world;
  if (W < 1 || W > kMaxPeers || ps->rank < 0 || ps->rank >= W || ps->cap < 1 || ps->cap >= (1 << 23) || ps->req == nullptr || ps->req_n == nullptr ||
      ps->peer_out == nullptr || ps->err == nullptr || ps->done == nullptr || (n > 0 && grad == nullptr))
    return SRM2_ERR_ARG;
  if (ps->ticket != 0 && (ps->peer_tickets == nullptr || ps->timeout_ns <= 0)) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || !aligned16(grad) || !aligned16(ps->req)) return SRM2_ERR_UNSUPPORTED;
  PeerPtrs pt{}, po{};
  for (int r = 0; r < W; ++r) {
    if (ps->ticket != 0 && ps->peer_tickets[r] == nullptr) return SRM2_ERR_ARG;
    if (r != ps->rank && (ps->peer_out[r] == nullptr || !aligned16(ps->peer_out[r]))) return SRM2_ERR_ARG;
    pt.p[r] = ps->ticket != 0 ? ps->peer_tickets[r] : nullptr;
    po.p[r] = ps->peer_out[r];
  }
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  // the number of requests is on the device; at most n / 2 of them (each names two or more of this rank's n rows)
  const int64_t items_max = (n / 2 + 1) * lpr;
  int64_t grid = (items_max + kPresumThreads - 1) / kPresumThreads;
  // One CTA per SM: the kernel runs beside the run-sum kernel of the step before, whose CTAs hold every register of the SMs
  // between them; every CTA here takes the place of two and a half of those for as long as it lives, and what bounds this
  // kernel is the latency of its dependent loads, not the number of its threads.
  if (grid > (int64_t)kSMs) grid = (int64_t)kSMs;
  if (grid < 1) grid = 1;
  srm2_presum_rows_kernel<<<(unsigned)grid, kPresumThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      grad, n, lpr, shift, (int)D, (int)W, (int)ps->rank, (uint32_t)ps->cap, static_cast<const uint4*>(ps->req), ps->req_n, po, ps->err, pt,
      (unsigned long long)ps->ticket, (long long)ps->timeout_ns, ps->done);
  return launch_status(1);
}
