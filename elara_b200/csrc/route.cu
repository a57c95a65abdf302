// Owner routing for row-sharded tables: lookups are grouped by owner rank (row_id mod world), keeping their order
// inside each group, and their gradient rows are gathered into one contiguous send buffer per owner.
//
// Stability matters: every owner later sums the lookups of a row in ascending GLOBAL lookup position; ranks hold
// consecutive slices of the batch, so a stable grouping on every rank plus concatenation in rank order on the owner
// reproduces the single-process order without shipping positions.
// Kernels: one stable counting pass of the radix sort (histogram, scatter; world <= 2048 owners) and a row gather
// that streams each gradient row once (D*4 bytes read + written per lookup, HBM bound).
#include "common.cuh"
#include "scan.cuh"
#include "sort.cuh"

namespace srm2 {

// out_lid[i] = ids[perm[i]] / world, out_grad[i,:] = grad[perm[i],:]; one thread per 16-byte lane.
__global__ void __launch_bounds__(256)
srm2_route_gather_kernel(const int64_t* __restrict__ ids, const float* __restrict__ grad, const uint32_t* __restrict__ perm,
                         int64_t n, int lpr, int shift, int D, int world, int64_t* __restrict__ out_lid,
                         float* __restrict__ out_grad) {
  const int64_t items = n * lpr;
  for (int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x; t < items; t += (int64_t)gridDim.x * 256) {
    int64_t i; int j4;
    if (shift >= 0) { i = t >> shift; j4 = (int)(t & (lpr - 1)); } else { i = t / lpr; j4 = (int)(t - i * lpr); }
    const uint32_t p = perm[i];
    const float4 g = ld_stream4(grad + (int64_t)p * D + j4 * 4);
    st_stream4(out_grad + t * 4, g);
    if (j4 == 0) { const int64_t id = ids[p]; out_lid[i] = id < 0 ? -1 : id / world; }
  }
}

// counts[o] = number of lookups owned by rank o: the digit totals of the single sort pass, or, when the histogram was
// scanned by the separate kernel, the difference of consecutive digit starts.
__global__ void srm2_route_counts_kernel(const uint32_t* __restrict__ hist, const uint32_t* __restrict__ dtot, int tiles, int world,
                                         int64_t n, int64_t* __restrict__ counts) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= world) return;
  if (dtot) { counts[o] = dtot[o]; return; }
  const int64_t lo = hist[(int64_t)o * tiles];
  const int64_t hi = (o + 1 < world) ? (int64_t)hist[(int64_t)(o + 1) * tiles] : n;
  counts[o] = hi - lo;
}

static size_t align_up_r(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int route_bits(int64_t world) { int b = 1; while (((int64_t)1 << b) < world) ++b; return b; }

static size_t route_layout(int64_t n, int64_t world, char* base, SortBuffers* sb) {
  const int tiles = sort_tiles(n > 0 ? n : 1);
  const int bits = route_bits(world);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up_r(off + bytes, 256); return o; };
  const size_t nn = (size_t)(n > 0 ? n : 1);
  const size_t o_ka = take(nn * 4), o_va = take(nn * 4), o_h = take(sort_hist_words(tiles, bits) * 4), o_dt = take(sort_dtot_words(tiles, bits, 1) * 4);
  if (sb) {
    auto u = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    sb->keyA = u(o_ka); sb->valA = u(o_va); sb->keyB = nullptr; sb->valB = nullptr; sb->hist = u(o_h); sb->dtot = u(o_dt); sb->tiles = tiles;
  }
  return off;
}

}  // namespace srm2

extern "C" size_t srm2_route_scratch_bytes(int64_t n, int64_t world) {
  if (n < 0 || world < 1) return 0;
  return srm2::route_layout(n, world, nullptr, nullptr);
}

extern "C" int srm2_route_by_owner(const int64_t* ids, const float* grad, int64_t n, int64_t D, int64_t world,
                                   int64_t* out_lid, float* out_grad, int64_t* out_counts, void* scratch,
                                   size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0 || world < 1 || out_counts == nullptr) return SRM2_ERR_ARG;
  if (n > 0 && (ids == nullptr || grad == nullptr || out_lid == nullptr || out_grad == nullptr)) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || world > (1 << kMaxRadixBits) || n >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (n > 0 && (!aligned16(grad) || !aligned16(out_grad))) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < route_layout(n, world, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    if (note_cuda(cudaMemsetAsync(out_counts, 0, (size_t)world * 8, st))) return SRM2_ERR_CUDA;
    return SRM2_OK;
  }
  SortBuffers sb;
  route_layout(n, world, static_cast<char*>(scratch), &sb);
  const uint32_t *skey = nullptr, *perm = nullptr;
  int launches = 0;
  const uint32_t* hb = nullptr;
  if (note_cuda(cudaMemsetAsync(sb.dtot, 0, sort_dtot_words(sb.tiles, route_bits(world), 1) * 4, st))) return SRM2_ERR_CUDA;
  const int rc = radix_sort_by_key(ids, n, nullptr, (int)world, 0, route_bits(world), 1, sb, &skey, &perm, &hb, &launches, st);
  if (rc != SRM2_OK) return rc;
  srm2_route_counts_kernel<<<(unsigned)((world + 255) / 256), 256, 0, st>>>(sb.hist, hb, sb.tiles, (int)world, n, out_counts);
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  const int64_t items = n * lpr;
  const int grid = (int)((items + 255) / 256 < (int64_t)kSMs * 16 ? (items + 255) / 256 : (int64_t)kSMs * 16);
  srm2_route_gather_kernel<<<grid, 256, 0, st>>>(ids, grad, perm, n, lpr, shift, (int)D, (int)world, out_lid, out_grad);
  return launch_status(launches + 2);
}

// ---------------------------------------------------------------------------------------------------------
// Routing fused with the exchange: instead of gathering into a local send buffer and handing that to a collective,
// the gather kernel stores every routed lookup straight into its owner's receive buffer over NVLink (peer pointers;
// plain stores, no multicast).  The only other traffic is the W x W matrix of lookup counts, which every rank
// publishes into every rank's copy the same way.  Two stream-ordered barriers of the caller's choice (any collective on
// the same stream) separate: counts published | rows dispatched | receive buffers read.
//   plan     : stable grouping by owner (sort pass) -> permutation + per-owner counts           (this rank only)
//   publish  : counts -> row `rank` of every rank's count matrix
//   dispatch : row offset in owner d's buffer = sum of counts[s][d] over ranks s < rank, plus the lookup's index in
//              this rank's group for d; rows and local ids are written there.  Receivers see their lookups in rank
//              order, each rank's part in its original order: the global lookup order.
namespace srm2 {

constexpr int kMaxPeers = 16;
struct PeerPtrs { void* p[kMaxPeers]; };

__global__ void srm2_route_publish_kernel(const int64_t* __restrict__ counts, PeerPtrs cmat, int rank, int world) {
  const int d = threadIdx.x;
  if (d >= world) return;
  const int64_t c = counts[d];
  for (int r = 0; r < world; ++r) static_cast<int64_t*>(cmat.p[r])[rank * world + d] = c;
}

__global__ void __launch_bounds__(256)
srm2_route_dispatch_kernel(const int64_t* __restrict__ ids, const float* __restrict__ grad, const uint32_t* __restrict__ perm,
                           const uint32_t* __restrict__ owner_sorted, int64_t n, int lpr, int shift, int D, int world, int rank,
                           const int64_t* __restrict__ cmat, PeerPtrs lid_peers, PeerPtrs grad_peers, int64_t cap,
                           int64_t* __restrict__ n_recv, uint32_t* __restrict__ err) {
  __shared__ int64_t s_start[kMaxPeers], s_base[kMaxPeers];
  if (threadIdx.x < world) {
    const int d = threadIdx.x;
    int64_t start = 0, base = 0;
    for (int e = 0; e < d; ++e) start += cmat[rank * world + e];      // first index of owner d in this rank's grouping
    for (int s = 0; s < rank; ++s) base += cmat[s * world + d];       // rows that lower ranks send to owner d
    s_start[d] = start; s_base[d] = base;
    if (blockIdx.x == 0 && d == rank) {
      int64_t tot = 0;
      for (int s = 0; s < world; ++s) tot += cmat[s * world + rank];
      *n_recv = tot;
      if (tot > cap) atomicOr(err, 1u);
    }
  }
  __syncthreads();
  const int64_t items = n * lpr;
  const int64_t stride = (int64_t)gridDim.x * 256;
  constexpr int U = 8;                                 // rows in flight per thread
  for (int64_t t0 = (int64_t)blockIdx.x * 256 + threadIdx.x; t0 < items; t0 += stride * U) {
    float4 g[U]; int64_t r[U]; uint32_t dd[U]; int j4s[U]; int64_t lid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t t = t0 + u * stride;
      r[u] = -1;
      if (t < items) {
        int64_t i; int j4;
        if (shift >= 0) { i = t >> shift; j4 = (int)(t & (lpr - 1)); } else { i = t / lpr; j4 = (int)(t - i * lpr); }
        const uint32_t d = owner_sorted[i];
        if (d < (uint32_t)world) {
          const int64_t rr = s_base[d] + (i - s_start[d]);
          if (rr >= cap) { atomicOr(err, 1u); }
          else {
            const uint32_t p = perm[i];
            g[u] = ld_stream4(grad + (int64_t)p * D + j4 * 4);
            lid[u] = 0;
            if (j4 == 0) { const int64_t id = ids[p]; lid[u] = id < 0 ? -1 : id / world; }
            r[u] = rr; dd[u] = d; j4s[u] = j4;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (r[u] >= 0) {
        *reinterpret_cast<float4*>(static_cast<float*>(grad_peers.p[dd[u]]) + r[u] * D + j4s[u] * 4) = g[u];
        if (j4s[u] == 0) static_cast<int64_t*>(lid_peers.p[dd[u]])[r[u]] = lid[u];
      }
    }
  }
}

// ---- the same dispatch with the copy engines of the SMs (bulk asynchronous copies) ---------------------------------
// One warp per CTA, one CTA per SM.  Lane l of a warp owns one routed lookup of a batch of 32: it issues a bulk copy
// of the lookup's gradient row from HBM into the warp's shared-memory stage (completion counted on the stage's
// mbarrier) and, once the batch has landed, a bulk copy from shared memory to the owner's receive buffer (peer memory,
// no multicast).  Three stages keep two batches of loads in flight per SM.  The warp issues a few instructions per
// 512-byte row and holds 48 KB of shared memory, so the shard update of the previous step keeps nearly all of every SM
// while the rows move.  Every wait is bounded: if an mbarrier does not complete within kTmaSpinLimit polls the kernel
// records err |= 4, drains its own copy groups and returns.
constexpr int kTmaStages = 3;
constexpr int kTmaRows = 32;
constexpr uint32_t kTmaSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

__global__ void __launch_bounds__(32)
srm2_route_dispatch_tma_kernel(const int64_t* __restrict__ ids, const float* __restrict__ grad, const uint32_t* __restrict__ perm,
                               const uint32_t* __restrict__ owner_sorted, int64_t n, int D, int world, int rank,
                               const int64_t* __restrict__ cmat, PeerPtrs lid_peers, PeerPtrs grad_peers, int64_t cap,
                               int64_t* __restrict__ n_recv, uint32_t* __restrict__ err) {
  extern __shared__ __align__(128) unsigned char stage_mem[];      // [kTmaStages][kTmaRows][row bytes]
  __shared__ __align__(8) uint64_t bar[kTmaStages];
  __shared__ int64_t s_start[kMaxPeers], s_base[kMaxPeers];
  const int lane = threadIdx.x;
  const uint32_t row_bytes = (uint32_t)D * 4u;
  if (lane < world) {
    const int d = lane;
    int64_t start = 0, base = 0;
    for (int e = 0; e < d; ++e) start += cmat[rank * world + e];
    for (int q = 0; q < rank; ++q) base += cmat[q * world + d];
    s_start[d] = start; s_base[d] = base;
    if (blockIdx.x == 0 && d == rank) {
      int64_t tot = 0;
      for (int q = 0; q < world; ++q) tot += cmat[q * world + rank];
      *n_recv = tot;
      if (tot > cap) atomicOr(err, 1u);
    }
  }
  if (lane == 0) {
    for (int q = 0; q < kTmaStages; ++q) mbar_init(&bar[q], 1u);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  // this CTA's contiguous share of the routed order, in batches of 32
  int64_t per = (n + gridDim.x - 1) / gridDim.x; per = (per + kTmaRows - 1) / kTmaRows * kTmaRows;
  const int64_t lo = (int64_t)blockIdx.x * per, hi = lo + per < n ? lo + per : n;
  const int64_t nb = hi > lo ? (hi - lo + kTmaRows - 1) / kTmaRows : 0;
  char* dst[kTmaStages];
  bool pending[kTmaStages];                              // a batch of loads is in flight into this stage
#pragma unroll
  for (int q = 0; q < kTmaStages; ++q) pending[q] = false;
  bool failed = false;

  auto issue_load = [&](int64_t b, int st) {
    const int64_t i = lo + b * kTmaRows + lane;
    bool valid = i < hi;
    uint32_t d = 0, p = 0; int64_t r = 0;
    if (valid) {
      d = owner_sorted[i];
      valid = d < (uint32_t)world;
      if (valid) { r = s_base[d] + (i - s_start[d]); if (r >= cap) { atomicOr(err, 1u); valid = false; } }
      if (valid) p = perm[i];
    }
    const unsigned vm = __ballot_sync(0xffffffffu, valid);
    if (lane == 0) mbar_expect_tx(&bar[st], (uint32_t)__popc(vm) * row_bytes);
    __syncwarp();
    dst[st] = nullptr;
    pending[st] = true;
    if (valid) {
      bulk_load(stage_mem + ((size_t)st * kTmaRows + lane) * row_bytes, grad + (int64_t)p * D, row_bytes, &bar[st]);
      const int64_t id = ids[p];
      static_cast<int64_t*>(lid_peers.p[d])[r] = id < 0 ? -1 : id / world;
      dst[st] = static_cast<char*>(grad_peers.p[d]) + r * (int64_t)row_bytes;
    }
  };

#pragma unroll
  for (int q = 0; q < kTmaStages - 1; ++q)
    if (q < nb) issue_load(q, q);
  for (int64_t b0 = 0; b0 < nb && !failed; b0 += kTmaStages) {
    const uint32_t parity = (uint32_t)((b0 / kTmaStages) & 1);
#pragma unroll
    for (int st = 0; st < kTmaStages; ++st) {
      const int64_t b = b0 + st;
      if (b >= nb || failed) break;
      uint32_t spins = 0;
      while (!mbar_try_wait(&bar[st], parity)) {
        if (++spins > kTmaSpinLimit) { failed = true; break; }
      }
      failed = __any_sync(0xffffffffu, failed);
      if (failed) break;
      pending[st] = false;
      if (dst[st] != nullptr) bulk_store(dst[st], stage_mem + ((size_t)st * kTmaRows + lane) * row_bytes, row_bytes);
      bulk_commit();
      // refill the stage that batch b-1 was stored from: its reads of shared memory must be over
      constexpr int kPrev = kTmaStages - 1;
      const int rs = (st + kPrev) % kTmaStages;
      if (b + kPrev < nb) { bulk_wait_read<1>(); issue_load(b + kPrev, rs); }
    }
  }
  if (failed) {
    // give the loads that are still in flight a bounded chance to land before the shared memory is given back
    if (lane == 0) atomicOr(err, 4u);
#pragma unroll
    for (int st = 0; st < kTmaStages; ++st) {
      if (!pending[st]) continue;
      for (uint32_t spins = 0; spins < kTmaSpinLimit; ++spins)
        if (mbar_try_wait(&bar[st], 0u) || mbar_try_wait(&bar[st], 1u)) break;
    }
  }
  bulk_wait_all();
}

}  // namespace srm2

extern "C" int srm2_route_plan(const int64_t* ids, int64_t n, int64_t world, int64_t* out_counts, void* scratch,
                               size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || world < 1 || out_counts == nullptr || (n > 0 && ids == nullptr)) return SRM2_ERR_ARG;
  if (world > kMaxPeers || n >= ((int64_t)1 << 31)) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < route_layout(n, world, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 0) return note_cuda(cudaMemsetAsync(out_counts, 0, (size_t)world * 8, st));
  SortBuffers sb;
  route_layout(n, world, static_cast<char*>(scratch), &sb);
  int launches = 0;
  const uint32_t *skey = nullptr, *perm = nullptr, *dt = nullptr;
  if (note_cuda(cudaMemsetAsync(sb.dtot, 0, sort_dtot_words(sb.tiles, route_bits(world), 1) * 4, st))) return SRM2_ERR_CUDA;
  const int rc = radix_sort_by_key(ids, n, nullptr, (int)world, 0, route_bits(world), 1, sb, &skey, &perm, &dt, &launches, st);
  if (rc != SRM2_OK) return rc;
  srm2_route_counts_kernel<<<(unsigned)((world + 255) / 256), 256, 0, st>>>(sb.hist, dt, sb.tiles, (int)world, n, out_counts);
  return launch_status(launches + 1);
}

extern "C" int srm2_route_publish(const int64_t* counts, void* const* peer_cmat, int64_t rank, int64_t world, srm2_stream_t stream) {
  using namespace srm2;
  if (counts == nullptr || peer_cmat == nullptr || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return SRM2_ERR_ARG;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) { if (peer_cmat[r] == nullptr) return SRM2_ERR_ARG; pp.p[r] = peer_cmat[r]; }
  srm2_route_publish_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(counts, pp, (int)rank, (int)world);
  return launch_status(1);
}

extern "C" int srm2_route_dispatch(const int64_t* ids, const float* grad, int64_t n, int64_t D, int64_t world, int64_t rank,
                                   const int64_t* cmat, void* const* peer_lid, void* const* peer_grad, int64_t cap,
                                   int64_t* n_recv, uint32_t* err, int use_tma, void* scratch, size_t scratch_bytes,
                                   srm2_stream_t stream) {
  using namespace srm2;
  if (n < 0 || D <= 0 || world < 1 || world > kMaxPeers || rank < 0 || rank >= world || cap < 0) return SRM2_ERR_ARG;
  if (cmat == nullptr || peer_lid == nullptr || peer_grad == nullptr || n_recv == nullptr || err == nullptr) return SRM2_ERR_ARG;
  if (n > 0 && (ids == nullptr || grad == nullptr)) return SRM2_ERR_ARG;
  if ((D & 3) != 0 || (n > 0 && !aligned16(grad))) return SRM2_ERR_UNSUPPORTED;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < route_layout(n, world, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  PeerPtrs pl{}, pg{};
  for (int r = 0; r < world; ++r) {
    if (peer_lid[r] == nullptr || peer_grad[r] == nullptr || !aligned16(peer_grad[r])) return SRM2_ERR_ARG;
    pl.p[r] = peer_lid[r]; pg.p[r] = peer_grad[r];
  }
  SortBuffers sb;
  route_layout(n, world, static_cast<char*>(scratch), &sb);     // keyA / valA hold the owners and the permutation of srm2_route_plan
  const int lpr = (int)(D / 4);
  const int shift = (lpr & (lpr - 1)) == 0 ? __builtin_ctz(lpr) : -1;
  const int64_t items = n * lpr;
  // a small grid: the kernel is bound by the NVLink stores, and it runs in the shadow of the previous step's shard
  // update, which should keep most of every SM
  int grid = (int)((items + 255) / 256 < (int64_t)kSMs * 2 ? (items + 255) / 256 : (int64_t)kSMs * 2);
  if (grid < 1) grid = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t tma_smem = (size_t)kTmaStages * kTmaRows * D * 4;
  if (use_tma && n > 0 && D * 4 <= 1024) {
    if (tma_smem > 48 * 1024 &&
        note_cuda(cudaFuncSetAttribute(srm2_route_dispatch_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tma_smem)))
      return SRM2_ERR_CUDA;
    const int64_t batches = (n + kTmaRows - 1) / kTmaRows;
    const int tgrid = (int)(batches < kSMs ? batches : kSMs);
    srm2_route_dispatch_tma_kernel<<<tgrid, 32, tma_smem, st>>>(ids, grad, sb.valA, sb.keyA, n, (int)D, (int)world, (int)rank, cmat, pl, pg,
                                                               cap, n_recv, err);
    return launch_status(1);
  }
  srm2_route_dispatch_kernel<<<grid, 256, 0, st>>>(ids, grad, sb.valA, sb.keyA, n, lpr, shift, (int)D, (int)world, (int)rank, cmat, pl, pg,
                                                  cap, n_recv, err);
  return launch_status(1);
}
