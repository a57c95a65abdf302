// ELARA state-directory update on the GPU: row codes (I / L_c / M), log-entry ids and steps, MAT slots, pool-slot
// residency and resident histories, with the two sync-free allocators (free stack + bump pointer for log ids, bump
// pointer for MAT slots).
//
// Replaces the reference's ATen op chains elara_dir_a / elara_dir_b (srm2/csrc/elara_dir.cpp:50-110, ~65 small library
// kernels per plan step) and the pool-slot admissions in between (srm2/elara.py:358-366) by seven fused kernels.
// Every id and slot is assigned by the same rule in the same order — rank of a request = its position among the valid
// requests of the call, free stack popped from the top, then the bump pointer — so directory state and returned ids are
// identical to the reference's.  Where the reference redirects masked-out lanes to "trash" elements (loc[R],
// ent[R*K..], lstep[Lcap], lfree[Lcap], pstep[Cdyn]) these kernels simply do not write: trash contents are unspecified
// in the reference as well (duplicate-index writes).
//
// All work is integer gather/scatter on a few thousand to a few hundred thousand items per call: latency-bound, a
// handful of microseconds per kernel; the figure of merit is the launch count and the time per plan step.
// Ranks come from block-local exclusive scans plus per-CTA prefixes that the last CTA to finish computes (no separate
// scan launch, no waiting between CTAs).  Indices handed in by the caller are range-checked; a violation sets a bit in
// the status word instead of touching memory.
#include "common.cuh"
#include "scan.cuh"

namespace srm2 {

constexpr int kDirT = 256;

struct DirSnap {            // written by the last CTA of a "prep" kernel, read by the "apply" kernels of the same call
  int64_t old_nf, old_top, old_mat;   // allocator state before this call's requests
  int64_t n_alloc, used, n_free, n_mat;
  uint32_t done; uint32_t status;     // finished-CTA counter (returns to 0); sticky error bits
};

constexpr uint32_t kErrRow = 1, kErrSlot = 2, kErrLog = 4;

struct DirScratch {
  DirSnap* snap;
  uint32_t *offA, *offM, *offF;       // [items] block-local exclusive offsets
  uint32_t *bA, *bM, *bF;             // [blocks] per-CTA totals, then exclusive prefixes
  int8_t* c0; int8_t* jv;             // [items] admission log count and resident history length of evicted slots
};

static size_t align_up_d(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t dir_layout(int64_t items, char* base, DirScratch* s) {
  const size_t it = (size_t)(items > 0 ? items : 1), nb = (it + kDirT - 1) / kDirT + 1;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up_d(off + bytes, 256); return o; };
  const size_t o_sn = take(sizeof(DirSnap));
  const size_t o_a = take(it * 4), o_m = take(it * 4), o_f = take(it * 4);
  const size_t o_ba = take(nb * 4), o_bm = take(nb * 4), o_bf = take(nb * 4);
  const size_t o_c0 = take(it), o_j = take(it);
  if (s) {
    auto u = [&](size_t o) { return reinterpret_cast<uint32_t*>(base + o); };
    s->snap = reinterpret_cast<DirSnap*>(base + o_sn);
    s->offA = u(o_a); s->offM = u(o_m); s->offF = u(o_f); s->bA = u(o_ba); s->bM = u(o_bm); s->bF = u(o_bf);
    s->c0 = reinterpret_cast<int8_t*>(base + o_c0); s->jv = reinterpret_cast<int8_t*>(base + o_j);
  }
  return off;
}

__device__ __forceinline__ bool row_ok(const srm2_dir_state& d, int64_t r) { return r >= 0 && r < d.R; }
__device__ __forceinline__ bool slot_ok(const srm2_dir_state& d, int64_t s) { return s >= 0 && s < d.n0 + d.Cdyn; }

// searchsorted(toff, row, right=True) - 1 (srm2/csrc/elara_dir.cpp:46-48)
__device__ __forceinline__ int64_t table_of(const srm2_dir_state& d, int64_t row) {
  int64_t lo = 0, hi = d.T;
  while (lo < hi) { const int64_t mid = (lo + hi) >> 1; if (d.toff[mid] <= row) lo = mid + 1; else hi = mid; }
  return lo - 1;
}

// Log id of allocation rank `rank` (srm2/csrc/elara_dir.cpp:13-17): free stack from the top, then the bump pointer.
__device__ __forceinline__ int64_t log_id(const srm2_dir_state& d, int64_t rank, int64_t nf, int64_t top) {
  return rank < nf ? (int64_t)d.lfree[nf - 1 - rank] : top + rank - nf;
}

// ---------------------------------------------------------------------------------------------- call A
// Replay inputs (elara_dir.cpp:57-59) and resident-history recording of pool hits (:61-71) in one launch:
// threads [0, nL*K) gather, threads [nL*K, nL*K + nh) record.
__global__ void __launch_bounds__(kDirT)
srm2_dir_gather_hits_kernel(srm2_dir_state d, const int64_t* __restrict__ hs, int64_t nh, const int64_t* __restrict__ L_row,
                            const int32_t* __restrict__ L_cnt, int64_t nL, int32_t step, int32_t* __restrict__ L_steps,
                            int32_t* __restrict__ L_ids, int64_t* __restrict__ hrec_dyn, int64_t* __restrict__ hrec_j,
                            DirSnap* __restrict__ snap) {
  const int64_t t = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  const int64_t K = d.K;
  if (t < nL * K) {
    const int64_t i = t / K, k = t - i * K;
    const int64_t row = L_row[i];
    int32_t e = -1;
    if (row_ok(d, row)) e = d.ent[row * K + k]; else atomicOr(&snap->status, kErrRow);
    int32_t st = 0;
    if (e >= 0) { if (e <= d.Lcap) st = d.lstep[e]; else atomicOr(&snap->status, kErrLog); }
    L_steps[t] = st;
    L_ids[t] = k < L_cnt[i] ? e : -1;
    return;
  }
  const int64_t i = t - nL * K;
  if (i >= nh) return;
  const int64_t sl = hs[i];
  if (!slot_ok(d, sl)) { atomicOr(&snap->status, kErrSlot); hrec_dyn[i] = d.Cdyn; hrec_j[i] = 0; return; }
  const bool dyn = sl >= d.n0;
  const int64_t c0 = d.adm_c0[sl], j = d.rj[sl];
  const bool ok = d.rok[sl] != 0;
  const bool rec = d.evl && dyn && ok && (c0 + j) < K;
  hrec_dyn[i] = rec ? sl - d.n0 : d.Cdyn;
  hrec_j[i] = rec ? j : 0;
  if (rec) d.pstep[(sl - d.n0) * K + j] = step;
  d.rj[sl] = (int8_t)(j + (rec ? 1 : 0));
  d.rok[sl] = (int8_t)(ok && !(dyn && !rec));
}

// Publishes block totals; the last CTA to finish turns them into exclusive prefixes and returns true in that CTA
// (with the grand totals in tot[3]).
__device__ __forceinline__ bool publish_and_scan3(uint32_t tA, uint32_t tM, uint32_t tF, uint32_t* bA, uint32_t* bM, uint32_t* bF,
                                                  uint32_t* done, int nblocks, uint32_t* ws, uint32_t (&tot)[3]) {
  __shared__ bool last;
  if (threadIdx.x == 0) {
    bA[blockIdx.x] = tA; bM[blockIdx.x] = tM; bF[blockIdx.x] = tF;
    __threadfence();
    last = atomicAdd(done, 1u) == (uint32_t)(nblocks - 1);
  }
  __syncthreads();
  if (!last) return false;
  __threadfence();
  uint32_t ca = 0, cm = 0, cf = 0;
  for (int base = 0; base < nblocks; base += kDirT) {
    const int i = base + threadIdx.x;
    const uint32_t va = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bA)[i] : 0u;
    const uint32_t vm = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bM)[i] : 0u;
    const uint32_t vf = i < nblocks ? reinterpret_cast<volatile uint32_t*>(bF)[i] : 0u;
    uint32_t t0, t1, t2;
    const uint32_t xa = block_exclusive_scan<kDirT>(va, ws, &t0);
    const uint32_t xm = block_exclusive_scan<kDirT>(vm, ws, &t1);
    const uint32_t xf = block_exclusive_scan<kDirT>(vf, ws, &t2);
    if (i < nblocks) { bA[i] = ca + xa; bM[i] = cm + xm; bF[i] = cf + xf; }
    ca += t0; cm += t1; cf += t2;
  }
  tot[0] = ca; tot[1] = cm; tot[2] = cf;
  return true;
}

// The allocator bookkeeping of one call (elara_dir.cpp:18-19, 31, 42), by thread 0 of the last CTA.
__device__ __forceinline__ void commit_allocators(srm2_dir_state& d, DirSnap* snap, int64_t n_alloc, int64_t n_mat, int64_t n_free) {
  const int64_t nf = *d.n_lfree, top = *d.log_top, mat = *d.mat_top;
  const int64_t used = n_alloc < nf ? n_alloc : nf;
  snap->old_nf = nf; snap->old_top = top; snap->old_mat = mat;
  snap->n_alloc = n_alloc; snap->used = used; snap->n_free = n_free; snap->n_mat = n_mat;
  *d.log_top = top + (n_alloc - used);
  *d.n_lfree = nf - used + n_free;
  *d.live = *d.live + n_alloc - n_free;
  *d.mat_top = mat + n_mat;
  snap->done = 0u;
}

// Eviction representation, part 1 (elara_dir.cpp:73-80, 89-92): per evicted slot the row, whether its history goes back
// to the log (rep), and the three request counts (log ids to allocate, MAT slot needed, log ids to release).
__global__ void __launch_bounds__(kDirT)
srm2_dir_evict_prep_kernel(srm2_dir_state d, const int64_t* __restrict__ ev_slot, int64_t nev, int64_t* __restrict__ ev_row,
                           uint8_t* __restrict__ rep, int64_t* __restrict__ ev_dyn, DirScratch s, int nblocks) {
  __shared__ uint32_t ws[33];
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  const int64_t K = d.K;
  uint32_t a = 0, m = 0, f = 0;
  if (i < nev) {
    const int64_t sl = ev_slot[i];
    int64_t row = -1; int64_t c0 = -1, j = 0; bool rp = false;
    if (slot_ok(d, sl)) {
      row = d.slot_row[sl]; c0 = d.adm_c0[sl]; j = d.rj[sl];
      if (row_ok(d, row)) {
        rp = d.evl && d.rok[sl] != 0 && (c0 + j) <= (int64_t)d.kthr[table_of(d, row)];
        d.slot_of[row] = -1;
      } else { atomicOr(&s.snap->status, kErrRow); row = -1; }
      d.slot_row[sl] = -1;
    } else atomicOr(&s.snap->status, kErrSlot);
    ev_row[i] = row; rep[i] = rp; ev_dyn[i] = sl - d.n0;
    s.c0[i] = (int8_t)c0; s.jv[i] = (int8_t)j;
    if (row >= 0) {
      if (rp) a = (uint32_t)(j < 0 ? 0 : (j > K ? K : j));
      else {
        m = d.loc[row] < 0;
        const int64_t cnt = c0 > 0 ? c0 : 0;
        for (int64_t k = 0; k < K; ++k) f += (k < cnt) && d.ent[row * K + k] >= 0;
      }
    }
  }
  uint32_t tA, tM, tF;
  const uint32_t ea = block_exclusive_scan<kDirT>(a, ws, &tA);
  const uint32_t em = block_exclusive_scan<kDirT>(m, ws, &tM);
  const uint32_t ef = block_exclusive_scan<kDirT>(f, ws, &tF);
  if (i < nev) { s.offA[i] = ea; s.offM[i] = em; s.offF[i] = ef; }
  uint32_t tot[3];
  if (publish_and_scan3(tA, tM, tF, s.bA, s.bM, s.bF, &s.snap->done, nblocks, ws, tot) && threadIdx.x == 0)
    commit_allocators(d, s.snap, tot[0], tot[1], tot[2]);
}

// Eviction representation, part 2 (elara_dir.cpp:81-90, 93): log ids for the resident histories that return to the log,
// MAT slots for the rows that materialise, row codes.
__global__ void __launch_bounds__(kDirT)
srm2_dir_evict_alloc_kernel(srm2_dir_state d, int64_t nev, const int64_t* __restrict__ ev_row, const uint8_t* __restrict__ rep,
                            const int64_t* __restrict__ ev_dyn, int64_t* __restrict__ evl_ids, int64_t* __restrict__ evf_slots,
                            DirScratch s) {
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  if (i >= nev) return;
  const int64_t K = d.K;
  const int64_t row = ev_row[i];
  const bool rp = rep[i] != 0;
  const int64_t c0 = s.c0[i], j = s.jv[i];
  const int64_t nf = s.snap->old_nf, top = s.snap->old_top;
  const int64_t rankA = (int64_t)s.bA[blockIdx.x] + s.offA[i];
  for (int64_t k = 0; k < K; ++k) {
    int64_t id = -1;
    if (row >= 0 && rp && k < j) {
      id = log_id(d, rankA + k, nf, top);
      if (id >= 0 && id < d.Lcap) {
        d.ent[row * K + (c0 > 0 ? c0 : 0) + k] = (int32_t)id;
        d.lstep[id] = d.pstep[ev_dyn[i] * K + k];
      } else atomicOr(&s.snap->status, kErrLog);
    }
    evl_ids[i * K + k] = id;
  }
  if (row < 0) { evf_slots[i] = d.trash; return; }
  const int64_t cur = d.loc[row];
  const bool nw = !rp && cur < 0;
  const int64_t sl = nw ? s.snap->old_mat + (int64_t)s.bM[blockIdx.x] + s.offM[i] : cur;
  if (nw) d.loc[row] = (int32_t)sl;
  evf_slots[i] = rp ? d.trash : sl;
  int64_t c = c0 + j; if (c > 127) c = 127;
  d.code[row] = rp ? (int8_t)c : (int8_t)d.MAT;
}

// Release of log entries (elara_dir.cpp:23-34) for rows[i] with cnt[i] entries (cnt8 != nullptr: the evictions of call
// A, where rows that return to the log release nothing and the others release max(c0, 0); else cnt64 of call B).
// Runs after every id of the call has been popped: pushes start at the new top of the free stack.
__global__ void __launch_bounds__(kDirT)
srm2_dir_release_kernel(srm2_dir_state d, int64_t n, const int64_t* __restrict__ rows, const uint8_t* __restrict__ rep,
                        const int8_t* __restrict__ cnt8, const int64_t* __restrict__ cnt64, DirScratch s) {
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  if (i >= n) return;
  const int64_t K = d.K;
  const int64_t row = rows[i];
  if (!row_ok(d, row)) return;
  int64_t cnt;
  if (cnt8) { cnt = rep[i] ? 0 : (cnt8[i] > 0 ? cnt8[i] : 0); } else cnt = cnt64[i];
  int64_t dst = s.snap->old_nf - s.snap->used + (int64_t)s.bF[blockIdx.x] + s.offF[i];
  for (int64_t k = 0; k < K; ++k) {
    const int32_t e = d.ent[row * K + k];
    if (k < cnt && e >= 0) {
      if (dst >= 0 && dst < d.Lcap) d.lfree[dst] = e; else atomicOr(&s.snap->status, kErrLog);
      ++dst;
      d.ent[row * K + k] = -1;
    }
  }
}

// ------------------------------------------------------------------------------------------ admissions
// Pool-slot admissions (srm2/elara.py:358-366): rows adm_rows take slots adm_slots; the first lazy_n come from states
// I / L and start a resident history at `step`.
__global__ void __launch_bounds__(kDirT)
srm2_dir_admit_kernel(srm2_dir_state d, const int64_t* __restrict__ adm_rows, const int64_t* __restrict__ adm_slots,
                      int64_t n_adm, int64_t lazy_n, int32_t step, DirSnap* __restrict__ snap) {
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  if (i >= n_adm) return;
  const int64_t r = adm_rows[i], sl = adm_slots[i];
  if (!row_ok(d, r)) { atomicOr(&snap->status, kErrRow); return; }
  if (!slot_ok(d, sl)) { atomicOr(&snap->status, kErrSlot); return; }
  const bool il = i < lazy_n, lazy = il && d.evl;
  d.slot_of[r] = (int32_t)sl; d.slot_row[sl] = r;
  d.adm_c0[sl] = il ? d.code[r] : (int8_t)-1;
  d.rj[sl] = (int8_t)lazy; d.rok[sl] = (int8_t)lazy;
  if (lazy && sl >= d.n0) d.pstep[(sl - d.n0) * d.K] = step;
}

// ---------------------------------------------------------------------------------------------- call B
// Appends (elara_dir.cpp:102-106): row a_rows[i] gets one new log id (rank i) at entry a_k[i]; compactions, part 1
// (:107-108): MAT slot needed / entries to release per row, scanned like the evictions.  One launch for both; the last
// CTA commits the allocator state of the whole call.
__global__ void __launch_bounds__(kDirT)
srm2_dir_append_prep_kernel(srm2_dir_state d, const int64_t* __restrict__ a_rows, const int64_t* __restrict__ a_k, int64_t na,
                            const int64_t* __restrict__ c_rows, const int64_t* __restrict__ c_cnt, int64_t nc, int32_t step,
                            int64_t* __restrict__ a_ids, DirScratch s, int nblocks) {
  __shared__ uint32_t ws[33];
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  const int64_t K = d.K;
  if (i < na) {
    const int64_t nf = *d.n_lfree, top = *d.log_top;     // not yet changed: the commit happens after every CTA is done
    const int64_t id = log_id(d, i, nf, top);
    const int64_t row = a_rows[i], k = a_k[i];
    a_ids[i] = id;
    if (!row_ok(d, row) || k < 0 || k >= K) atomicOr(&s.snap->status, kErrRow);
    else if (id < 0 || id >= d.Lcap) atomicOr(&s.snap->status, kErrLog);
    else { d.ent[row * K + k] = (int32_t)id; d.lstep[id] = step; d.code[row] = (int8_t)(k + 1); }
  }
  uint32_t m = 0, f = 0;
  if (i < nc) {
    const int64_t row = c_rows[i];
    if (row_ok(d, row)) {
      m = d.loc[row] < 0;
      const int64_t cnt = c_cnt[i];
      for (int64_t k = 0; k < K; ++k) f += (k < cnt) && d.ent[row * K + k] >= 0;
    } else atomicOr(&s.snap->status, kErrRow);
  }
  uint32_t tA, tM, tF;
  block_exclusive_scan<kDirT>(0u, ws, &tA);
  const uint32_t em = block_exclusive_scan<kDirT>(m, ws, &tM);
  const uint32_t ef = block_exclusive_scan<kDirT>(f, ws, &tF);
  if (i < nc) { s.offM[i] = em; s.offF[i] = ef; }
  uint32_t tot[3];
  if (publish_and_scan3(0u, tM, tF, s.bA, s.bM, s.bF, &s.snap->done, nblocks, ws, tot) && threadIdx.x == 0)
    commit_allocators(d, s.snap, na, tot[1], tot[2]);
}

// Compactions, part 2 (elara_dir.cpp:36-44, 108): MAT slots and codes.
__global__ void __launch_bounds__(kDirT)
srm2_dir_compact_kernel(srm2_dir_state d, const int64_t* __restrict__ c_rows, int64_t nc, int64_t* __restrict__ c_slots,
                        DirScratch s) {
  const int64_t i = (int64_t)blockIdx.x * kDirT + threadIdx.x;
  if (i >= nc) return;
  const int64_t row = c_rows[i];
  if (!row_ok(d, row)) { c_slots[i] = -1; return; }
  const int64_t cur = d.loc[row];
  const bool nw = cur < 0;
  const int64_t sl = nw ? s.snap->old_mat + (int64_t)s.bM[blockIdx.x] + s.offM[i] : cur;
  if (nw) d.loc[row] = (int32_t)sl;
  c_slots[i] = sl;
  d.code[row] = (int8_t)d.MAT;
}

static int dir_check(const srm2_dir_state* d) {
  if (d == nullptr) return SRM2_ERR_ARG;
  if (d->R <= 0 || d->K <= 0 || d->K > 64 || d->Lcap <= 0 || d->n0 < 0 || d->Cdyn < 0 || d->T <= 0) return SRM2_ERR_ARG;
  const void* ptrs[] = {d->code, d->loc, d->ent, d->lstep, d->lfree, d->n_lfree, d->log_top, d->mat_top, d->live, d->adm_c0, d->rj,
                        d->pstep, d->kthr, d->toff, d->slot_of, d->slot_row, d->rok};
  for (const void* p : ptrs) if (p == nullptr) return SRM2_ERR_ARG;
  return SRM2_OK;
}

static int blocks_for(int64_t items) { return (int)((items + kDirT - 1) / kDirT); }

}  // namespace srm2

extern "C" size_t srm2_dir_scratch_bytes(int64_t max_items) { return srm2::dir_layout(max_items, nullptr, nullptr); }

extern "C" int srm2_dir_a(const srm2_dir_state* st_, const int64_t* hs, int64_t nh, const int64_t* L_row, const int32_t* L_cnt,
                          int64_t nL, const int64_t* ev_slot, int64_t nev, int64_t step, int32_t* L_steps, int32_t* L_ids,
                          int64_t* hrec_dyn, int64_t* hrec_j, int64_t* ev_row, uint8_t* rep, int64_t* evl_ids,
                          int64_t* evf_slots, int64_t* ev_dyn, void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  int rc = dir_check(st_);
  if (rc) return rc;
  if (nh < 0 || nL < 0 || nev < 0) return SRM2_ERR_ARG;
  if ((nh && (!hs || !hrec_dyn || !hrec_j)) || (nL && (!L_row || !L_cnt || !L_steps || !L_ids)) ||
      (nev && (!ev_slot || !ev_row || !rep || !evl_ids || !evf_slots || !ev_dyn))) return SRM2_ERR_ARG;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < dir_layout(nev, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  srm2_dir_state d = *st_;
  DirScratch s;
  dir_layout(nev, static_cast<char*>(scratch), &s);
  if (note_cuda(cudaMemsetAsync(s.snap, 0, sizeof(DirSnap), st))) return SRM2_ERR_CUDA;
  int launches = 0;
  const int64_t t1 = nL * d.K + nh;
  if (t1 > 0) {
    srm2_dir_gather_hits_kernel<<<blocks_for(t1), kDirT, 0, st>>>(d, hs, nh, L_row, L_cnt, nL, (int32_t)step, L_steps, L_ids, hrec_dyn,
                                                                 hrec_j, s.snap);
    ++launches;
  }
  if (nev > 0) {
    const int nb = blocks_for(nev);
    srm2_dir_evict_prep_kernel<<<nb, kDirT, 0, st>>>(d, ev_slot, nev, ev_row, rep, ev_dyn, s, nb);
    srm2_dir_evict_alloc_kernel<<<nb, kDirT, 0, st>>>(d, nev, ev_row, rep, ev_dyn, evl_ids, evf_slots, s);
    srm2_dir_release_kernel<<<nb, kDirT, 0, st>>>(d, nev, ev_row, rep, s.c0, nullptr, s);
    launches += 3;
  }
  return launch_status(launches);
}

extern "C" int srm2_dir_admit(const srm2_dir_state* st_, const int64_t* adm_rows, const int64_t* adm_slots, int64_t n_adm,
                              int64_t lazy_n, int64_t step, void* scratch, size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  int rc = dir_check(st_);
  if (rc) return rc;
  if (n_adm < 0 || lazy_n < 0 || lazy_n > n_adm) return SRM2_ERR_ARG;
  if (n_adm == 0) return SRM2_OK;
  if (!adm_rows || !adm_slots) return SRM2_ERR_ARG;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < dir_layout(0, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  DirScratch s;
  dir_layout(0, static_cast<char*>(scratch), &s);
  srm2_dir_admit_kernel<<<blocks_for(n_adm), kDirT, 0, static_cast<cudaStream_t>(stream)>>>(*st_, adm_rows, adm_slots, n_adm, lazy_n,
                                                                                           (int32_t)step, s.snap);
  return launch_status(1);
}

extern "C" int srm2_dir_b(const srm2_dir_state* st_, const int64_t* a_rows, const int64_t* a_k, int64_t na, const int64_t* c_rows,
                          const int64_t* c_cnt, int64_t nc, int64_t step, int64_t* a_ids, int64_t* c_slots, void* scratch,
                          size_t scratch_bytes, srm2_stream_t stream) {
  using namespace srm2;
  int rc = dir_check(st_);
  if (rc) return rc;
  if (na < 0 || nc < 0) return SRM2_ERR_ARG;
  if ((na && (!a_rows || !a_k || !a_ids)) || (nc && (!c_rows || !c_cnt || !c_slots))) return SRM2_ERR_ARG;
  const int64_t items = na > nc ? na : nc;
  if (items == 0) return SRM2_OK;
  if (scratch == nullptr || !aligned16(scratch) || scratch_bytes < dir_layout(items, nullptr, nullptr)) return SRM2_ERR_SCRATCH;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  srm2_dir_state d = *st_;
  DirScratch s;
  dir_layout(items, static_cast<char*>(scratch), &s);
  // only the counter and the request totals are cleared: the status word is sticky across the calls of a plan step
  if (note_cuda(cudaMemsetAsync(s.snap, 0, offsetof(DirSnap, status), st))) return SRM2_ERR_CUDA;
  const int nb = blocks_for(items);
  srm2_dir_append_prep_kernel<<<nb, kDirT, 0, st>>>(d, a_rows, a_k, na, c_rows, c_cnt, nc, (int32_t)step, a_ids, s, nb);
  int launches = 1;
  if (nc > 0) {
    srm2_dir_compact_kernel<<<blocks_for(nc), kDirT, 0, st>>>(d, c_rows, nc, c_slots, s);
    srm2_dir_release_kernel<<<blocks_for(nc), kDirT, 0, st>>>(d, nc, c_rows, nullptr, nullptr, c_cnt, s);
    launches += 2;
  }
  return launch_status(launches);
}

extern "C" int srm2_dir_status(const void* scratch, uint32_t* status_out /* device or pinned host, 4 bytes */, srm2_stream_t stream) {
  using namespace srm2;
  if (scratch == nullptr || status_out == nullptr) return SRM2_ERR_ARG;
  DirScratch s;
  dir_layout(0, const_cast<char*>(static_cast<const char*>(scratch)), &s);
  return note_cuda(cudaMemcpyAsync(status_out, &s.snap->status, 4, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}
