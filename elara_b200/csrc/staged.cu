// A window of optimizer steps enqueued as a pipeline of stages on five streams, seven with more than one rank (see
// srm2_staged in the header).
// Pure host code: it makes the library's own calls and orders them with CUDA events.  Written in C++ because a step is
// about twenty launches and an interpreted host loop needs longer to issue them than the GPU needs to run them.
#include "common.cuh"

static_assert(sizeof(srm2_staged) == 66 * 8, "srm2_staged: every member is 8 bytes wide");

namespace srm2 {
namespace {

constexpr int kRing = 16;          // events per stage; every dependency reaches back fewer steps than this
constexpr int kSets = 4;           // buffer sets: dedup, sort, descriptors and sums each hold one

struct Staged {
  const srm2_staged& a;
  cudaStream_t xs, ds, so, ix, ms, pr = nullptr, pl = nullptr;
  bool pull, presum;
  int rc = SRM2_OK;
  explicit Staged(const srm2_staged& s) : a(s), pull(s.world > 1), presum(s.world > 1 && s.presum_cap > 0) {
    xs = static_cast<cudaStream_t>(a.streams[0]); ds = static_cast<cudaStream_t>(a.streams[1]);
    so = static_cast<cudaStream_t>(a.streams[2]); ix = static_cast<cudaStream_t>(a.streams[3]); ms = static_cast<cudaStream_t>(a.streams[4]);
    if (pull) { pr = static_cast<cudaStream_t>(a.streams[5]); pl = static_cast<cudaStream_t>(a.streams[6]); }
  }
  cudaEvent_t ev(int stage, int64_t k) const { return static_cast<cudaEvent_t>(a.events[stage * kRing + (int)(k % kRing)]); }
  bool ok() const { return rc == SRM2_OK; }
  void trace(int64_t k, int stage, int end, cudaStream_t st) {
    if (a.trace_events) cuda(cudaEventRecord(static_cast<cudaEvent_t>(a.trace_events[k * 14 + stage * 2 + end]), st));
  }
  void check(int r) { if (rc == SRM2_OK && r != SRM2_OK) rc = r; }
  void cuda(cudaError_t e) { if (rc == SRM2_OK && note_cuda(e)) rc = SRM2_ERR_CUDA; }
  void barrier(cudaStream_t st) {
    *a.ticket += 1;
    check(srm2_peer_barrier(a.peer_tickets, a.rank, a.world, (uint64_t)*a.ticket, a.err, a.timeout_ns, nullptr, st));
  }

  srm2_presum presum_base() const {
    srm2_presum ps{};
    ps.world = a.world; ps.rank = a.rank; ps.cap = a.presum_cap; ps.timeout_ns = a.timeout_ns; ps.err = a.err;
    return ps;
  }

  // stage 5 (world > 1): the routing plan of step k — local work, on a stream of its own.  Two scratch sets:
  // the names stage of step k-2 was the last reader of this one.
  char* route_set(int64_t k) const { return static_cast<char*>(a.route_scr) + (k & 1) * a.route_scr_bytes; }
  void plan(int64_t k) {
    if (k >= 2) cuda(cudaStreamWaitEvent(pl, ev(0, k - 2), 0));
    check(srm2_route_plan(static_cast<const int64_t*>(a.ids[k]), a.n_k[k], a.world, a.counts + (k & 1) * a.world, route_set(k), (size_t)a.route_scr_bytes, pl));
    cuda(cudaEventRecord(ev(5, k), pl));
  }
  // stage 0: names of step k to their owners
  void exchange(int64_t k) {
    const int64_t R = a.n_recv_bufs, S = a.n_slots, W = a.world, b = k % R, nk = a.n_k[k];
    cuda(cudaStreamWaitEvent(xs, ev(5, k), 0));
    if (k >= R) cuda(cudaStreamWaitEvent(xs, ev(3, k - R), 0));          // these receive buffers have been consumed
    if (k >= S) cuda(cudaStreamWaitEvent(xs, ev(4, k - S), 0));          // nobody enters the barrier while it still reads the slot
    trace(k, 0, 0, xs);
    // counts to every rank and the first barrier in one kernel: count matrices complete, receive buffers and slot free
    *a.ticket += 1;
    check(srm2_route_publish_barrier(a.counts + (k & 1) * W, a.peer_cmat + b * W, a.peer_tickets, a.rank, W, (uint64_t)*a.ticket, a.err, a.timeout_ns, xs));
    float* slot = a.slot[k % S];
    if (a.grads[k] != slot && nk > 0)
      cuda(cudaMemcpyAsync(slot, a.grads[k], (size_t)nk * a.D * 4, cudaMemcpyDeviceToDevice, xs));
    // names to their owners; the last CTA is the second barrier: every name has arrived, every slot is filled
    *a.ticket += 1;
    check(srm2_route_dispatch_ids(static_cast<const int64_t*>(a.ids[k]), nk, W, a.rank, a.cmat[b], a.peer_lid + b * W, a.peer_src + b * W, a.cap,
                                  a.n_recv + (k & 7), a.err, a.peer_tickets, (uint64_t)*a.ticket, a.timeout_ns, route_set(k), (size_t)a.route_scr_bytes, xs));
    trace(k, 0, 1, xs);
    cuda(cudaEventRecord(ev(0, k), xs));
  }
  // stage 1
  void dedup(int64_t k) {
    const int64_t q = k % kSets;
    if (pull) cuda(cudaStreamWaitEvent(ds, ev(0, k), 0));
    if (k >= kSets) cuda(cudaStreamWaitEvent(ds, ev(4, k - kSets), 0));  // this buffer set has been consumed
    trace(k, 1, 0, ds);
    const int64_t* ids = pull ? a.recv_lid[k % a.n_recv_bufs] : static_cast<const int64_t*>(a.ids[k]);
    const int64_t* n_dev = pull ? a.n_recv + (k & 7) : nullptr;
    check(srm2_unique_inverse_nd_i64(ids, a.n, n_dev, a.n_rows, a.u[q], a.cap_u, a.inv[q], a.counts_out + 2 * k, a.scr_u, (size_t)a.scr_u_bytes, ds));
    trace(k, 1, 1, ds);
    cuda(cudaEventRecord(ev(1, k), ds));
  }
  // stages 2 and 3: the index half of the fused reduce in its two parts
  void index(int64_t k, int part) {
    const int64_t q = k % kSets;
    cudaStream_t st = part == SRM2_INDEX_SORT ? so : ix;
    cuda(cudaStreamWaitEvent(st, ev(part == SRM2_INDEX_SORT ? 1 : 2, k), 0));
    trace(k, part == SRM2_INDEX_SORT ? 2 : 3, 0, st);
    const uint32_t* src = pull ? a.recv_src[k % a.n_recv_bufs] : nullptr;
    const int64_t* n_dev = pull ? a.n_recv + (k & 7) : nullptr;
    const int64_t cap_u = a.cap_u < a.n ? a.cap_u : a.n;
    check(srm2_reduce_adam_index(a.u[q], src, a.inv[q], a.n, n_dev, a.D, -1, a.counts_out + 2 * k, cap_u, part, a.scr_s[q], (size_t)a.scr_s_bytes, st));
    if (presum && part == SRM2_INDEX_DESCRIPTORS) {
      trace(k, 5, 0, st);
      // requests for sums prepared at the source: set k mod n_slots of every rank's request buffers (the sums of step
      // k - n_slots, their last reader, ended on every rank before anybody left the first barrier of this step's exchange)
      const int64_t set = k % a.n_slots;
      srm2_presum ps = presum_base();
      ps.peer_req = a.peer_req + set * a.world; ps.peer_req_n = a.peer_req_n + set * a.world; ps.req_count = a.req_count + set * 32;
      ps.peer_tickets = a.peer_tickets_req; *a.ticket += 1; ps.ticket = (uint64_t)*a.ticket;
      check(srm2_presum_request(a.n, n_dev, a.D, cap_u, a.scr_s[q], (size_t)a.scr_s_bytes, &ps, st));
      trace(k, 5, 1, st);
    }
    trace(k, part == SRM2_INDEX_SORT ? 2 : 3, 1, st);
    cuda(cudaEventRecord(ev(part == SRM2_INDEX_SORT ? 2 : 3, k), st));
  }
  // stage 6 (sums prepared at the source), between descriptors and sums on a stream of its own: this rank adds up what its
  // peers asked for out of the step's gradient slot and stores the sums into the peers' buffers; the kernel ends with a
  // barrier, so every rank's sums have arrived when the stage is complete.  It depends on gradients, but not on the table:
  // with the next step's gradients in place it runs while the run-sum kernel of the step before is still at work.
  // Three buffers of sums per rank: the stage of step k waits for this rank's sums stage of step k - 2, so it runs at most
  // two steps ahead, and its kernel starts behind the barrier of step k - 1 (same stream), which no rank entered before its
  // own sums stage of step k - 3 — the last reader of the buffer that is written now — had ended.
  void prepare_sums(int64_t k) {
    const int64_t set = k % a.n_slots;
    cuda(cudaStreamWaitEvent(pr, ev(3, k), 0));                            // the requests are complete (barrier of the descriptors stage)
    if (k >= 2) cuda(cudaStreamWaitEvent(pr, ev(4, k - 2), 0));
    trace(k, 6, 0, pr);
    srm2_presum ps = presum_base();
    ps.req = a.req[set]; ps.req_n = a.req_n[set]; ps.peer_out = a.peer_push + (k % 3) * a.world; ps.done = a.presum_done;
    ps.peer_tickets = a.peer_tickets_sum; *a.ticket += 1; ps.ticket = (uint64_t)*a.ticket;
    check(srm2_presum_rows_f32(a.slot[set], a.n_k[k], a.D, &ps, pr));
    trace(k, 6, 1, pr);
    cuda(cudaEventRecord(ev(6, k), pr));
  }
  // stage 4
  void sums(int64_t k) {
    const int64_t q = k % kSets;
    cuda(cudaStreamWaitEvent(ms, ev(3, k), 0));
    if (presum) cuda(cudaStreamWaitEvent(ms, ev(6, k), 0));                // every rank's prepared sums of this step have arrived
    trace(k, 4, 0, ms);
    float sc[8];
    check(srm2_adam_scalars(a.lr, a.b1, a.b2, a.eps, a.first_step + k, sc));
    if (a.stage_events) srm2_stage_events(a.stage_events[2 * k], a.stage_events[2 * k + 1]);
    const int64_t cap_u = a.cap_u < a.n ? a.cap_u : a.n;
    if (presum) {
      check(srm2_reduce_adam_apply_pull_f32(a.pool, a.u[q], a.peer_slot + (k % a.n_slots) * a.world, a.peer_out + (k % 3) * a.world, a.err, a.world, a.n,
                                            a.n_recv + (k & 7), a.D, -1, a.counts_out + 2 * k, cap_u, sc, a.scr_s[q], (size_t)a.scr_s_bytes, ms));
    } else if (pull)
      check(srm2_reduce_adam_apply_f32(a.pool, a.u[q], nullptr, a.peer_slot + (k % a.n_slots) * a.world, a.world, a.n, a.n_recv + (k & 7), a.D, -1,
                                       a.counts_out + 2 * k, cap_u, sc, a.scr_s[q], (size_t)a.scr_s_bytes, ms));
    else
      check(srm2_reduce_adam_apply_f32(a.pool, a.u[q], static_cast<const float*>(a.grads[k]), nullptr, 1, a.n, nullptr, a.D, -1, a.counts_out + 2 * k,
                                       cap_u, sc, a.scr_s[q], (size_t)a.scr_s_bytes, ms));
    trace(k, 4, 1, ms);
    cuda(cudaEventRecord(ev(4, k), ms));
  }

  int run() {
    const int64_t K = a.K;
    // the side streams start behind what the caller's stream has enqueued so far
    cudaEvent_t start = ev(4, kRing - 1);
    cuda(cudaEventRecord(start, ms));
    for (cudaStream_t st : {xs, ds, so, ix}) cuda(cudaStreamWaitEvent(st, start, 0));
    if (pull) { cuda(cudaStreamWaitEvent(pr, start, 0)); cuda(cudaStreamWaitEvent(pl, start, 0)); }
    // prologue; then every iteration enqueues one step of every stage, the oldest first, so that a stage only ever waits
    // for events that have been recorded by then
    for (int64_t k = 0; k < 5 && k < K && pull && ok(); ++k) {           // plan(k) overwrites what exchange(k-2) read
      plan(k);
      if (k >= 1 && k - 1 < 4) exchange(k - 1);
    }
    if (pull && K <= 4 && K >= 1 && ok()) exchange(K - 1);               // short windows: the last exchange of the prologue
    for (int64_t k = 0; k < 3 && k < K && ok(); ++k) dedup(k);
    for (int64_t k = 0; k < 2 && k < K && ok(); ++k) index(k, SRM2_INDEX_SORT);
    if (K > 0 && ok()) index(0, SRM2_INDEX_DESCRIPTORS);
    if (presum && K > 0 && ok()) prepare_sums(0);
    for (int64_t k = 0; k < K && ok(); ++k) {
      sums(k);
      if (k + 1 < K && ok()) index(k + 1, SRM2_INDEX_DESCRIPTORS);
      if (presum && k + 1 < K && ok()) prepare_sums(k + 1);
      if (k + 2 < K && ok()) index(k + 2, SRM2_INDEX_SORT);
      if (k + 3 < K && ok()) dedup(k + 3);
      if (pull && k + 4 < K && ok()) exchange(k + 4);
      if (pull && k + 5 < K && ok()) plan(k + 5);
    }
    if (a.stage_events) srm2_stage_events(nullptr, nullptr);
    // join: what follows on the caller's stream sees the window complete
    if (K > 0) {
      int stage = 0;
      for (cudaStream_t st : {xs, ds, so, ix}) {
        cudaEvent_t j = ev(stage++, K);                                   // a ring entry nobody waits on any more
        cudaEventRecord(j, st); cudaStreamWaitEvent(ms, j, 0);
      }
      if (pull) {
        cudaEvent_t j = ev(6, K); cudaEventRecord(j, pr); cudaStreamWaitEvent(ms, j, 0);
        j = ev(5, K); cudaEventRecord(j, pl); cudaStreamWaitEvent(ms, j, 0);
      }
    }
    if (pull && ok()) barrier(ms);                                        // no rank returns while a peer may still read its slots
    return rc;
  }
};

}  // namespace
}  // namespace srm2

extern "C" int srm2_staged_steps(const srm2_staged* a) {
  using namespace srm2;
  if (a == nullptr || a->K < 0 || a->n < 0 || a->D <= 0 || a->ids == nullptr || a->grads == nullptr || a->n_k == nullptr || a->streams == nullptr ||
      a->events == nullptr || a->pool == nullptr || a->counts_out == nullptr)
    return SRM2_ERR_ARG;
  for (int q = 0; q < 4; ++q)
    if (a->u[q] == nullptr || a->inv[q] == nullptr || a->scr_s[q] == nullptr) return SRM2_ERR_ARG;
  if (a->world > 1) {
    if (a->world > 16 || a->rank < 0 || a->rank >= a->world || a->n_recv_bufs < 4 || a->n_recv_bufs >= 16 || a->n_slots < 4 || a->n_slots >= 16 ||
        a->timeout_ns <= 0 || a->route_scr == nullptr || a->counts == nullptr || a->err == nullptr || a->n_recv == nullptr || a->cmat == nullptr ||
        a->recv_lid == nullptr || a->recv_src == nullptr || a->peer_cmat == nullptr || a->peer_lid == nullptr || a->peer_src == nullptr ||
        a->slot == nullptr || a->peer_slot == nullptr || a->peer_tickets == nullptr || a->ticket == nullptr)
      return SRM2_ERR_ARG;
    if (a->presum_cap > 0 && (a->peer_req == nullptr || a->peer_req_n == nullptr || a->req == nullptr || a->req_n == nullptr || a->req_count == nullptr ||
                              a->peer_push == nullptr || a->peer_out == nullptr || a->peer_tickets_req == nullptr || a->peer_tickets_sum == nullptr ||
                              a->presum_done == nullptr))
      return SRM2_ERR_ARG;
  } else {
    for (int64_t k = 0; k < a->K; ++k)
      if (a->n_k[k] != a->n) return SRM2_ERR_ARG;
  }
  Staged s(*a);
  return s.run();
}
