/*
 * srm2_b200 — C ABI of the B200 (sm_100a) kernels for the sparse-optimizer path of ELARA's srm2 package.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the parameter comment says "host".
 *   - Nothing here allocates, frees or synchronises; scratch memory is passed in by the caller.
 *   - Every call enqueues its kernels on `stream` (a cudaStream_t passed as void*; NULL = legacy default
 *     stream) of the CURRENT device and returns immediately.
 *   - Return value: SRM2_OK (0) or a negative SRM2_ERR_* code; srm2_status_string() names it.  Argument
 *     errors are detected on the host before anything is enqueued.
 *   - fp32 arithmetic is IEEE round-to-nearest, one rounding per operation, no FMA contraction, in the
 *     operation order of the reference, so results are bit-identical to the reference's CPU and GPU paths.
 *
 * Each entry point names the reference interface it stands in for (paths relative to the reference project).
 */
#ifndef SRM2_B200_H
#define SRM2_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SRM2_OK 0
#define SRM2_ERR_ARG (-1)         /* null pointer, negative size, inconsistent arguments            */
#define SRM2_ERR_UNSUPPORTED (-2) /* a size outside what the kernels are built for                  */
#define SRM2_ERR_SCRATCH (-3)     /* scratch buffer too small (see the *_scratch_bytes functions)   */
#define SRM2_ERR_CUDA (-4)        /* the CUDA runtime refused a launch; see srm2_last_cuda_error()  */
#define SRM2_ERR_LIMIT (-5)       /* larger than the fixed scratch of srm2_unique_inverse_noalloc_i64 */

typedef void* srm2_stream_t;

/* library identification: major*10000 + minor*100 + patch */
int srm2_version(void);
const char* srm2_status_string(int status);
/* text of the last CUDA runtime error seen by this thread inside the library ("" if none) */
const char* srm2_last_cuda_error(void);
/* number of kernels this library has enqueued in this process so far (all threads) */
int64_t srm2_launch_count(void);
/* Instrumentation for benchmarks: while set (per calling thread), srm2_segment_reduce_f32 / srm2_reduce_adam_f32 record
 * the cudaEvent_t `begin` before and `end` after their gradient-streaming kernels, on the call's stream.  Pass NULL, NULL
 * to clear.  No counterpart in the reference. */
int srm2_stage_events(void* begin /* cudaEvent_t */, void* end /* cudaEvent_t */);

/* Self-check of the library's short correctly-rounded fp32 division / square-root sequences (the arithmetic inside the
 * Adam, replay and fused reduce kernels) against the compiler's IEEE operations, run on the current GPU.  No
 * counterpart in the reference (its kernels use the compiler's operations directly); used by the tests.
 *   what     SRM2_VERIFY_SQRT: every float bit pattern in [lo, hi) inside the guarded range;
 *            SRM2_VERIFY_DIV_HARD: divisor significands 2^23 + [lo, hi), every dividend whose quotient lies within `param`
 *            odd steps of a rounding midpoint (divisors with more than 8 trailing zero bits are left to DIV_ALL);
 *            SRM2_VERIFY_DIV_ALL: all 2^23 dividend significands against divisors 2^23 + (i << param), i in [lo, hi);
 *            SRM2_VERIFY_DIV_RANDOM: hi - lo pseudo-random pairs of seed lo over the guarded exponent range;
 *            SRM2_VERIFY_ADAM: hi - lo pseudo-random whole Adam steps on four elements (seed lo), the packed step against the
 *            plain IEEE step; param 0 = operands as in training, 1 = arbitrary bit patterns (NaN, infinities, subnormals)
 *   variant  which sequence (square root: 1..3; division: number of residual corrections, 1 or 2); the kernels use
 *            variant 1 of each (ignored by SRM2_VERIFY_ADAM)
 *   out5     device uint64[5], ACCUMULATED into (zero it first): cases tested, mismatches, bits of the first mismatching
 *            dividend and divisor, divisors whose refined reciprocal is off by more than 2^-22 (DIV_HARD) */
#define SRM2_VERIFY_SQRT 0
#define SRM2_VERIFY_DIV_HARD 1
#define SRM2_VERIFY_DIV_ALL 2
#define SRM2_VERIFY_DIV_RANDOM 3
#define SRM2_VERIFY_ADAM 4
int srm2_verify_exact(int what, uint64_t lo, uint64_t hi, int variant, int param, uint64_t* out5, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Adam scalars.  Replaces `adam_scalars` of the reference's host extension
 * (srm2/csrc/srm2_cpu.cpp:13-20 make_scalars, :255-257 export; called at srm2/ops.py:64 and srm2/gpu_ops.py:87).
 * out (host) = {lr, b1, 1-b1, b2, 1-b2, 1-b1^step, 1-b2^step, eps}, each evaluated in double, rounded to float once.
 */
int srm2_adam_scalars(double lr, double b1, double b2, double eps, int64_t step, float out[8] /* host */);

/* ---------------------------------------------------------------------------------------------------------
 * Row-sparse Adam.  Replaces `gpu_adam` / Triton `_adam_rows` (srm2/ops.py:42-67); same arithmetic as the
 * reference's `cpu_adam` (srm2/csrc/srm2_cpu.cpp:22-56).
 *   pool   [C,3,D] fp32, row record = w[D] m[D] v[D]; updated in place for the rows named in `slots`
 *   slots  [n] int32 (slots_is_i64 == 0) or int64 (!= 0), DISTINCT row indices into pool
 *   grad   [n,D] fp32 contiguous; row i belongs to slots[i]
 *   sc     (host) the 8 scalars of srm2_adam_scalars
 * n == 0 is a no-op.
 */
int srm2_adam_rows_f32(float* pool, const void* slots, int slots_is_i64, const float* grad, int64_t n, int64_t D,
                       const float sc[8] /* host */, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Counter-hash row initialisation.  Replaces `init_rows` / Triton `_init_rows` (srm2/gpu_ops.py:15-48).
 *   out [n,3,D] fp32: w = (u*2-1)*bound with u = (fmix32(key ^ seed) >> 8) * 2^-24,
 *                     key = (uint32)(row*D + j) ^ fmix32((uint32)(row >> 32) + seed); m = v = 0
 *   rows [n] int64;  seed = the reference's integer seed truncated to 32 bits.
 */
int srm2_init_rows_f32(float* out, const int64_t* rows, int64_t n, int64_t D, uint32_t seed, float bound,
                       srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Exact replay of up to K logged gradients into freshly initialised rows.
 * Replaces `replay_rows` / Triton `_replay` (srm2/gpu_ops.py:51-99).
 *   out   [n,3,D]            rows [n] int64
 *   logs  flat [sum(cnt), D] fp32; the entries of row i start at offs[i] (int64 [n])
 *   steps [n,K] int32 logical step of each entry;  cnt [n] int32 (0..K)
 *   table [table_rows, 8] fp32: Adam scalars per logical step (`ScalarTable.t`, srm2/gpu_ops.py:82-88)
 */
int srm2_replay_rows_f32(float* out, const int64_t* rows, const float* logs, const int64_t* offs, const int32_t* steps,
                         const int32_t* cnt, int64_t n, int64_t D, int64_t K, uint32_t seed, float bound,
                         const float* table, int64_t table_rows, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Dedup of row ids from a bounded universe.  Replaces the driver's `torch.unique(ids, return_inverse=True)`
 * (srm2/train.py:352; ids are global row ids in [0, R), srm2/train.py:205-214).
 *   ids       [n] int64 in [0, n_rows)
 *   uniq      [uniq_cap] int64: the distinct ids in ascending order (entries past the count are untouched;
 *             ranks >= uniq_cap are dropped, so uniq_cap = min(n, n_rows) always suffices)
 *   inv       [n] int64: index of ids[p] in uniq (-1 for an id outside [0, n_rows))
 *   out_count [2] int64 (device): [0] = number of distinct ids, [1] = 1 if an id was out of range
 *   scratch   srm2_unique_scratch_bytes(n_rows) bytes, 256-byte aligned; contents need not be preserved
 * The result is a pure function of the input: no atomically assigned positions, no run-to-run variation.
 */
size_t srm2_unique_scratch_bytes(int64_t n_rows);
int srm2_unique_inverse_i64(const int64_t* ids, int64_t n, int64_t n_rows, int64_t* uniq, int64_t uniq_cap, int64_t* inv,
                            int64_t* out_count, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Segment-reduce of per-lookup gradients.  Replaces the driver's
 * `torch.ops.aten.embedding_dense_backward(grad, inv, n_unique, -1, False)` (srm2/train.py:429), in that
 * operator's CUDA summation order (torch 2.11.0): see elara_b200/csrc/segreduce.cu.
 *   grad [n,D] fp32 (D % 4 == 0, D <= 512, 16-byte aligned; n < 2,097,152);  inv [n] int64 in [0, n_unique)
 *   out  [n_unique, D] fp32; rows without lookups are zero
 *   n_unique      host value, used when n_unique_dev == NULL
 *   n_unique_dev  optional device int64: the count is read on the device (no host sync after a dedup);
 *                 max_unique then bounds it and sizes the scratch
 *   order         SRM2_ORDER_AUTO: the operator's rule (windows of 32 positions for n <= 3072, runs of 10 above);
 *                 SRM2_ORDER_RUNS / SRM2_ORDER_WINDOWS force one (a shard of a larger batch must use the order of the
 *                 whole batch)
 *   scratch       srm2_segment_scratch_bytes(n, max_unique or n_unique, D) bytes, 256-byte aligned
 */
#define SRM2_ORDER_AUTO 0
#define SRM2_ORDER_RUNS 1
#define SRM2_ORDER_WINDOWS 2
size_t srm2_segment_scratch_bytes(int64_t n, int64_t max_unique, int64_t D);
int srm2_segment_reduce_f32(const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t n_unique,
                            const int64_t* n_unique_dev, int64_t max_unique, int order, float* out, void* scratch,
                            size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Segment-reduce fused with row-sparse Adam: the two reference calls
 * `gW = embedding_dense_backward(...)` (srm2/train.py:429) and `gpu_adam(pool, slots, gW, ...)`
 * (srm2/ops.py:59-67) in one pass; gW is never written.  Same bits as the two calls in sequence.
 *   pool [C,3,D]; slots [n_unique] int64 distinct pool rows (slots[j] belongs to unique row j); other
 *   arguments as in srm2_segment_reduce_f32 and srm2_adam_rows_f32.
 */
int srm2_reduce_adam_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n, int64_t D,
                         int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, int order,
                         const float sc[8] /* host */, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Owner routing for row-sharded tables (rows owned by row_id mod world, local row = row_id div world).
 * No counterpart in the reference, which is single-GPU; it serves the row-sharded benchmark configuration.
 *   ids [n] int64 global row ids, grad [n,D] fp32
 *   out_lid  [n] int64: local row ids (row_id div world) grouped by owner rank 0..world-1, original order kept
 *            inside each group;  out_grad [n,D]: the gradient rows in the same order
 *   out_counts [world] int64 (device): lookups per owner
 *   scratch  srm2_route_scratch_bytes(n, world) bytes, 256-byte aligned
 */
size_t srm2_route_scratch_bytes(int64_t n, int64_t world);
int srm2_route_by_owner(const int64_t* ids, const float* grad, int64_t n, int64_t D, int64_t world, int64_t* out_lid,
                        float* out_grad, int64_t* out_counts, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * ELARA state directory (device-resident).  Field for field the reference's state vector
 * (srm2/csrc/elara_dir.cpp:8-11, built at srm2/elara.py:117-149, 275-277).  The struct itself lives on the host and
 * is passed by pointer; all array members are device pointers.
 */
typedef struct srm2_dir_state {
  int8_t* code;          /* [R]          row code: 0 = I, 1..K = L_c, MAT = M                              */
  int32_t* loc;          /* [R+1]        MAT slot of a row (-1 none); last element unused ("trash")        */
  int32_t* ent;          /* [(R+1)*K]    log-entry ids, row-major [R+1, K] (-1 empty); last row unused      */
  int32_t* lstep;        /* [Lcap+1]     logical step of each log entry                                     */
  int32_t* lfree;        /* [Lcap+1]     free stack of log ids                                              */
  int64_t* n_lfree;      /* [1]          entries on the free stack                                          */
  int64_t* log_top;      /* [1]          bump pointer of the log arena                                      */
  int64_t* mat_top;      /* [1]          bump pointer of the MAT arena                                      */
  int64_t* live;         /* [1]          live log entries                                                   */
  int8_t* adm_c0;        /* [C]          host log entries of the resident row at admission (-1: came from M) */
  int8_t* rj;            /* [C]          gradients recorded while resident                                  */
  int32_t* pstep;        /* [Cdyn+1, K]  steps of the resident history of each dynamic slot                 */
  const int8_t* kthr;    /* [T]          per-table materialisation threshold                                */
  const int64_t* toff;   /* [T]          first row of each table, ascending                                 */
  int32_t* slot_of;      /* [R]          pool slot of a row (-1 not resident)                               */
  int64_t* slot_row;     /* [C]          row held by a pool slot (-1 free)                                  */
  int8_t* rok;           /* [C]          resident history is complete (representable as log entries)        */
  int64_t R, K, Lcap, n0, Cdyn, MAT, trash, evl, T;   /* C = n0 + Cdyn; evl: evictions may return rows to L */
} srm2_dir_state;

/* scratch for the directory calls of one plan step; max_items >= max(nev, na, nc); 256-byte aligned; the SAME buffer
 * must be passed to srm2_dir_a, srm2_dir_admit, srm2_dir_b and srm2_dir_status of a step */
size_t srm2_dir_scratch_bytes(int64_t max_items);

/* Call A.  Replaces `elara_dir_a` (srm2/csrc/elara_dir.cpp:50-96; torch twin srm2/elara.py:285-343): replay inputs of
 * the L rows, resident-history recording of the pool hits, representation of the evicted slots (back to L with newly
 * allocated log ids, or to M with a MAT slot and release of their host log entries).
 *   in : hs [nh] int64 hit slots (distinct), L_row [nL] int64, L_cnt [nL] int32, ev_slot [nev] int64 (distinct), step
 *   out: L_steps [nL,K] int32, L_ids [nL,K] int32, hrec_dyn [nh] int64, hrec_j [nh] int64, ev_row [nev] int64,
 *        rep [nev] uint8/bool, evl_ids [nev,K] int64, evf_slots [nev] int64, ev_dyn [nev] int64 */
int srm2_dir_a(const srm2_dir_state* st /* host */, const int64_t* hs, int64_t nh, const int64_t* L_row, const int32_t* L_cnt,
               int64_t nL, const int64_t* ev_slot, int64_t nev, int64_t step, int32_t* L_steps, int32_t* L_ids,
               int64_t* hrec_dyn, int64_t* hrec_j, int64_t* ev_row, uint8_t* rep, int64_t* evl_ids, int64_t* evf_slots,
               int64_t* ev_dyn, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* Pool-slot admissions between the two calls.  Replaces the torch statements at srm2/elara.py:358-366:
 * adm_rows [n_adm] take adm_slots [n_adm]; the first lazy_n rows come from states I / L. */
int srm2_dir_admit(const srm2_dir_state* st /* host */, const int64_t* adm_rows, const int64_t* adm_slots, int64_t n_adm,
                   int64_t lazy_n, int64_t step, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* Call B.  Replaces `elara_dir_b` (srm2/csrc/elara_dir.cpp:98-110; torch twin srm2/elara.py:380-386): appends
 * (a_rows [na], entry index a_k [na] -> a_ids [na] int64) and compactions (c_rows [nc], c_cnt [nc] -> c_slots [nc]). */
int srm2_dir_b(const srm2_dir_state* st /* host */, const int64_t* a_rows, const int64_t* a_k, int64_t na, const int64_t* c_rows,
               const int64_t* c_cnt, int64_t nc, int64_t step, int64_t* a_ids, int64_t* c_slots, void* scratch,
               size_t scratch_bytes, srm2_stream_t stream);

/* Copies the step's sticky error word (bit 0: row index out of range, bit 1: pool slot out of range, bit 2: log id out
 * of range / arena overflow) to status_out (device or pinned host memory) on the stream.  The offending access was
 * skipped, never performed.  The reference has no counterpart: it indexes unchecked. */
int srm2_dir_status(const void* scratch, uint32_t* status_out, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Dedup for callers that cannot provide scratch memory.  No counterpart in the reference.
 *
 * Same inputs, outputs and results as srm2_unique_inverse_i64, but no scratch argument: the kernels work on a fixed
 * area inside the library image (a __device__ array of about 1 MiB that every GPU loading the library holds until the
 * process ends).  Meant for hosts that must not allocate device memory where they need the dedup — a process whose
 * memory cap is already spent on its tables, a loop that cannot take the device-wide synchronisation an allocation
 * may cause, a host whose device memory belongs to another allocator.  The entry point itself allocates and frees
 * nothing, on the device or through any library.
 *   - Limit: n_rows <= srm2_unique_noalloc_max_rows() (4,194,304); beyond it the call returns SRM2_ERR_LIMIT and
 *     enqueues nothing.
 *   - First use on a device: the first call made while a given device is current asks the CUDA runtime for the device
 *     address of the area (cudaGetSymbolAddress) and remembers it for that device.  Make that first call outside any
 *     stream capture.
 *   - The area is shared by every call in the process and keeps the previous call's contents; each call clears what it
 *     needs zeroed, on its own stream.  Two calls whose kernels may overlap on one GPU (different streams without an
 *     ordering between them, or different host threads) race on the area and give undefined results: order them.
 */
int64_t srm2_unique_noalloc_max_rows(void);
int srm2_unique_inverse_noalloc_i64(const int64_t* ids, int64_t n, int64_t n_rows, int64_t* uniq, int64_t uniq_cap,
                                    int64_t* inv, int64_t* out_count, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Owner routing fused with the exchange (no counterpart in the reference): routed lookups are stored directly into the
 * owners' receive buffers through peer pointers over NVLink (plain stores), so no send buffer and no collective moves
 * the payload.  world <= 16.  Call order per step, all on one stream, with a stream-ordered barrier across the ranks
 * (any collective on that stream) where marked:
 *   srm2_route_plan      this rank's stable grouping by owner; out_counts [world] int64 (device)
 *   srm2_route_publish   counts -> row `rank` of every rank's [world, world] int64 count matrix (peer_cmat: host array of
 *                        `world` device pointers, entry r = rank r's matrix)
 *   -- barrier --        every matrix is complete; every rank has reset the tail of its receive buffer
 *   srm2_route_dispatch  local ids (row_id div world) -> peer_lid[d] [cap] int64 and gradient rows -> peer_grad[d] [cap, D]
 *                        of each owner d, at the row offsets that give rank order; n_recv (device int64) = rows this rank
 *                        will receive; *err |= 1 if a receive buffer would overflow (those rows are not written).
 *                        use_tma != 0 (rows of at most 1 KiB): one warp per SM gathers the rows into shared memory with
 *                        cp.async and sends them with bulk asynchronous copies shared -> owner.
 *                        `scratch` must be the buffer srm2_route_plan was given.
 *   -- barrier --        every row has arrived
 * Receive buffers hold cap rows; fill their id part with -1 before the first barrier so that unused rows are ignored
 * by srm2_unique_inverse_i64 (inverse -1) and srm2_reduce_adam_f32.
 */
int srm2_route_plan(const int64_t* ids, int64_t n, int64_t world, int64_t* out_counts, void* scratch, size_t scratch_bytes,
                    srm2_stream_t stream);
int srm2_route_publish(const int64_t* counts, void* const* peer_cmat /* host */, int64_t rank, int64_t world, srm2_stream_t stream);
int srm2_route_dispatch(const int64_t* ids, const float* grad, int64_t n, int64_t D, int64_t world, int64_t rank,
                        const int64_t* cmat, void* const* peer_lid /* host */, void* const* peer_grad /* host */, int64_t cap,
                        int64_t* n_recv, uint32_t* err, int use_tma, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Pull form of the same exchange (no counterpart in the reference): the gradient rows stay in the buffer of the rank
 * that produced them (peer-accessible memory) and only the names of the lookups travel.  The owner's fused
 * segment-reduce + Adam reads each row from its source over NVLink while it sums, so the rows cross the link once and
 * are never written to or re-read from the owner's memory.
 *   srm2_route_plan, srm2_route_publish, -- barrier --   as above
 *   srm2_route_dispatch_ids   local ids -> peer_lid[d] [cap] int64 and codes (rank << 24) | position -> peer_src[d] [cap]
 *                             uint32 of each owner d, same offsets, n_recv and err as srm2_route_dispatch; n < 2^24.
 *   -- barrier --             every name has arrived
 *   srm2_unique_inverse_nd_i64 on the received ids, then
 *   srm2_reduce_adam_pull_f32 like srm2_reduce_adam_nd_f32 with order SRM2_ORDER_RUNS, except that lookup i's gradient
 *                             row is row (src_code[i] & 0xffffff) of peer_grad[src_code[i] >> 24] (host array of `world`
 *                             device pointers, 16-byte aligned, row stride D floats).
 *   -- barrier --             before any rank overwrites a gradient buffer that peers may still be reading
 */
/* Stream-ordered barrier across the ranks' GPUs for the "-- barrier --" marks above (no counterpart in the reference;
 * any collective on the stream serves as well, this one is a single one-warp kernel).  peer_tickets: host array of
 * `world` device pointers, entry r = rank r's array of 16 uint64 in peer-visible memory, zero before the first use.
 * `ticket` must grow by one with every barrier and be the same on every rank.  A rank whose peers do not arrive within
 * timeout_ns sets bit 1 (value 2) of *err and carries on: the wait is bounded, the caller must check *err.
 * Containment: *err is sticky, and a rank that leaves the barrier with *err != 0 writes 0 to *n_recv when n_recv is given
 * (the barrier behind the names of a step: pass that step's count of received lookups) — the update kernels of the step
 * then see an empty batch and leave the shard as it was.  The barrier fused into srm2_route_dispatch_ids does the same. */
int srm2_peer_barrier(void* const* peer_tickets /* host */, int64_t rank, int64_t world, uint64_t ticket, uint32_t* err,
                      int64_t timeout_ns, int64_t* n_recv /* or NULL */, srm2_stream_t stream);
/* Measurement aid (no counterpart in the reference): streams `bytes` from src — local memory or a peer's — with the
 * 16-byte asynchronous copies the fused reduce + Adam kernel uses for gradient rows, on every SM, and discards them.
 * Time it with events to get the read ceiling of that access path on this machine.  src 16-byte aligned; sink: any
 * device float (written only for one unlikely value of the checksum). */
int srm2_read_probe(const void* src, size_t bytes, float* sink, srm2_stream_t stream);
int srm2_route_dispatch_ids(const int64_t* ids, int64_t n, int64_t world, int64_t rank, const int64_t* cmat,
                            void* const* peer_lid /* host */, void* const* peer_src /* host */, int64_t cap, int64_t* n_recv,
                            uint32_t* err, void* const* peer_tickets /* host or NULL */, uint64_t ticket, int64_t timeout_ns,
                            void* scratch, size_t scratch_bytes, srm2_stream_t stream);
/* The two barriers of the exchange folded into its kernels (fewer launches, fewer NVLink round trips in the stream):
 *   srm2_route_plan_publish  = srm2_route_plan + srm2_route_publish + srm2_peer_barrier(ticket): the plan's last kernel
 *                              stores the counts into every rank's matrix and goes through the barrier;
 *   srm2_route_dispatch_ids with peer_tickets != NULL and ticket != 0: the last CTA to finish goes through the barrier
 *                              (srm2_peer_barrier semantics, same bounded wait and status bit). */
/*   srm2_route_publish_barrier = srm2_route_publish + srm2_peer_barrier for counts of a plan that ran earlier. */
int srm2_route_publish_barrier(const int64_t* counts, void* const* peer_cmat /* host */, void* const* peer_tickets /* host */,
                               int64_t rank, int64_t world, uint64_t ticket, uint32_t* err, int64_t timeout_ns, srm2_stream_t stream);
int srm2_route_plan_publish(const int64_t* ids, int64_t n, int64_t world, int64_t rank, int64_t* out_counts,
                            void* const* peer_cmat /* host */, void* const* peer_tickets /* host */, uint64_t ticket, uint32_t* err,
                            int64_t timeout_ns, void* scratch, size_t scratch_bytes, srm2_stream_t stream);
int srm2_reduce_adam_pull_f32(float* pool, const int64_t* slots, const float* const* peer_grad /* host */, int64_t world,
                              const uint32_t* src_code, const int64_t* inv, int64_t n, const int64_t* n_dev, int64_t D,
                              int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, const float sc[8] /* host */,
                              void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Variants whose lookup count lives on the device (no counterpart in the reference): n is an upper bound that sizes
 * grids and scratch, the kernels process min(n, *n_dev) lookups.  They let a receive buffer of fixed capacity be
 * consumed without reading its fill level on the host (row-sharded exchange).  n_dev == NULL behaves like the plain
 * entry points.  For SRM2_ORDER_AUTO the order is chosen from the bound n.
 */
int srm2_unique_inverse_nd_i64(const int64_t* ids, int64_t n, const int64_t* n_dev, int64_t n_rows, int64_t* uniq,
                               int64_t uniq_cap, int64_t* inv, int64_t* out_count, void* scratch, size_t scratch_bytes,
                               srm2_stream_t stream);
int srm2_reduce_adam_nd_f32(float* pool, const int64_t* slots, const float* grad, const int64_t* inv, int64_t n,
                            const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique,
                            int order, const float sc[8] /* host */, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * The fused segment-reduce + Adam in two halves (no counterpart in the reference).  Everything up to the run
 * descriptors depends on the lookups' row indices only, not on the gradients: a training loop that knows the ids of
 * the next batch ahead (data-loader prefetch) can run srm2_unique_inverse_* and srm2_reduce_adam_index for step s+1
 * on a second stream while srm2_reduce_adam_apply_f32 of step s streams the gradient rows.  The halves communicate
 * through `scratch` alone (same n, D, max_unique and scratch in both calls; order them with an event); use one scratch
 * buffer per step in flight.  Order of summation: SRM2_ORDER_RUNS.  Precondition: every unique row has at least one
 * lookup (as srm2_unique_inverse_* produces); a row without lookups is left unchanged by the split form.
 *   srm2_reduce_adam_index      src_code == NULL: lookup i's gradient is row i of `grad` given to the apply call;
 *                               src_code != NULL: pull form, see srm2_reduce_adam_pull_f32.
 *                               part: SRM2_INDEX_ALL, or the two parts as separate calls (again on streams of their own):
 *                               SRM2_INDEX_SORT (sort by unique row; needs inv) then
 *                               SRM2_INDEX_DESCRIPTORS (segment boundaries, plan, run descriptors; needs slots and src_code).
 *   srm2_reduce_adam_apply_f32  exactly one of grad (local rows) and peer_grad (host array of `world` device pointers)
 *                               is non-NULL and must match the index call.
 */
#define SRM2_INDEX_ALL 0
#define SRM2_INDEX_SORT 1
#define SRM2_INDEX_DESCRIPTORS 2
int srm2_reduce_adam_index(const int64_t* slots, const uint32_t* src_code, const int64_t* inv, int64_t n, const int64_t* n_dev,
                           int64_t D, int64_t n_unique, const int64_t* n_unique_dev, int64_t max_unique, int part, void* scratch,
                           size_t scratch_bytes, srm2_stream_t stream);
int srm2_reduce_adam_apply_f32(float* pool, const int64_t* slots, const float* grad, const float* const* peer_grad /* host */,
                               int64_t world, int64_t n, const int64_t* n_dev, int64_t D, int64_t n_unique,
                               const int64_t* n_unique_dev, int64_t max_unique, const float sc[8] /* host */, void* scratch,
                               size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Capacity-tier arenas in device memory.  Replace `cpu_gather` / `cpu_scatter` of the reference's host extension
 * (srm2/csrc/srm2_cpu.cpp:58-81) for arenas that live in HBM instead of host DRAM: the MAT arena [Mcap+1, 3, D] and the log
 * arena [Lcap+1, 1, D] of `ArenaStore` (srm2/elara.py:40-48), addressed by the physical ids the planner hands out.
 *   gather   out[i] [ncomp, D] = the first ncomp D-vectors of record ids[i] of arena [n_rec, W, D]
 *   scatter  the first Wc D-vectors of record ids[i] = src[i] [Wc, D]   (ids distinct, as the reference's are)
 * ids int64; an id outside [0, n_rec) is skipped and sets bit 0 of *bad (device uint32, may be NULL).  D % 4 == 0. */
int srm2_arena_gather_f32(float* out, const float* arena, const int64_t* ids, int64_t n, int64_t n_rec, int64_t W, int64_t ncomp,
                          int64_t D, uint32_t* bad, srm2_stream_t stream);
int srm2_arena_scatter_f32(float* arena, const float* src, const int64_t* ids, int64_t n, int64_t n_rec, int64_t W, int64_t Wc,
                           int64_t D, uint32_t* bad, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Executor update.  Replaces the GPU half of `ELARAExecutor.update` (srm2/elara.py:497-531: ~25 index_select /
 * index_put_ / index_copy_ / cat calls and three gpu_adam launches) by three kernels on one stream:
 *   hits   for every resident row: its gradient G[hit_pos[i]] is recorded as entry hrec_j[i] of history row hrec_dyn[i]
 *          (when evl != 0; glog is the [Cdyn+1, K, D] history tensor, row Cdyn = trash) and applied to pool[hit_slot[i]];
 *   pack   og [n_S + nNp + nLp, D]  = G[S_pos], G[N_pos[appended]], G[L_pos[appended]]
 *          of [nNc + nLc + nFn + n_evM, 3, D] = Adam(fullN[compacted]), Adam(fullL[compacted]), Adam(ff[not admitted]),
 *                                               pool[evM_slot]   (read after `hits`, before `admit`)
 *          oe [n_evl, D]            = glog.view(-1, D)[evl_src]
 *   admit  pool[N_adm_slot] = Adam(fullN[admitted]), pool[L_adm_slot] = Adam(fullL[admitted]), pool[F_adm_slot] =
 *          Adam(ff[admitted]); the gradients of the admitted N and L rows become entry 0 of history row adm_rec_dyn[k]
 *          (k counts the N admissions, then the L admissions) when evl != 0.
 * Rows of fullN / fullL / ff are ordered as the planner emits them: admitted, appended, compacted (N, L) and admitted,
 * not admitted (F) — the index ranges of `p.ix` in the reference.  fullN, fullL and ff are not modified.  Positions,
 * slots and history indices are int64.  sc: the eight scalars of srm2_adam_scalars for this step.  D % 4 == 0 and
 * 16-byte aligned float buffers, SRM2_ERR_UNSUPPORTED otherwise.  Every member is 8 bytes wide except sc. */
typedef struct srm2_update {
  int64_t D, K, evl;
  const float* G; float* pool; float* glog;
  float sc[8];
  const int64_t* hit_pos; const int64_t* hit_slot; const int64_t* hrec_dyn; const int64_t* hrec_j; int64_t n_hit;
  const int64_t* S_pos; int64_t n_S;
  const float* fullN; const int64_t* N_pos; int64_t nNa, nNp, nNc;
  const float* fullL; const int64_t* L_pos; int64_t nLa, nLp, nLc;
  const float* ff; const int64_t* F_pos; int64_t nFa, nFn;
  const int64_t* evM_slot; int64_t n_evM;
  const int64_t* evl_src; int64_t n_evl;
  const int64_t* N_adm_slot; const int64_t* L_adm_slot; const int64_t* F_adm_slot; const int64_t* adm_rec_dyn;
  float* og; float* of; float* oe;
} srm2_update;
int srm2_executor_update_f32(const srm2_update* u /* host */, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Fused assemble.  Replaces the body of `ELARAExecutor.assemble` (srm2/elara.py:479-489: torch.empty, init_rows,
 * replay_rows and ten index_select / index_copy_ calls) by one kernel.  W [n, D] receives one weight row per unique row of
 * the step from five sources, each given as (positions in W, source):
 *   resident rows      W[hit_pos[i]] = pool[hit_slot[i], 0]                      pool [C,3,D]
 *   never-touched rows fullN[i] = init of N_row[i] (as srm2_init_rows_f32);      W[N_pos[i]] = fullN[i,0]
 *   logged rows        fullL[i] = replay of L_row[i] (as srm2_replay_rows_f32);  W[L_pos[i]] = fullL[i,0]
 *   staged full rows   W[F_pos[i]] = ff[i,0]                                      ff [n_F,3,D]
 *   staged weights     W[S_pos[i]] = sw[i]                                        sw [n_S,D]
 * Positions and rows are int64; L_steps [n_L,K] and L_cnt [n_L] int32.  fullN [n_N,3,D] and fullL [n_L,3,D] are outputs
 * (the update step scatters them into the pool).  A position outside [0, n) is skipped.  D % 4 == 0, K <= 8 and 16-byte
 * aligned float buffers; SRM2_ERR_UNSUPPORTED otherwise (use the separate calls then).
 */
/* Forward gather of the step, the companion of srm2_assemble_f32 on the same stream: out[p] = W[inv[p]] for the n lookups
 * (replaces `torch.index_select(W, 0, inv)`, srm2/train.py:427).  W [n_rows, D] as just assembled (L2-resident), inv int64 [n]
 * (an index outside [0, n_rows) yields a zero row), out [n, D].  D % 4 == 0, 16-byte aligned buffers. */
int srm2_gather_rows_f32(float* out, const float* W, const int64_t* inv, int64_t n, int64_t n_rows, int64_t D, srm2_stream_t stream);
int srm2_assemble_f32(float* W, int64_t n, int64_t D, const float* pool, const int64_t* hit_pos, const int64_t* hit_slot,
                      int64_t n_hit, float* fullN, const int64_t* N_pos, const int64_t* N_row, int64_t n_N, uint32_t seed,
                      float bound, float* fullL, const int64_t* L_pos, const int64_t* L_row, const float* logs,
                      const int64_t* L_off, const int32_t* L_steps, const int32_t* L_cnt, int64_t n_L, int64_t K,
                      const float* table, int64_t table_rows, const float* ff, const int64_t* F_pos, int64_t n_F,
                      const float* sw, const int64_t* S_pos, int64_t n_S, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Classification and class partition of a step's unique rows.  Replaces, inside `ELARAPlanner.plan`, the expressions of
 * srm2/elara.py:214-219 (pool slot, hit, look-ahead membership, admission), :229-239 (code, table threshold, the
 * 10-way class of srm2/elara.py:32), :243 (class counts) and :258 (order = stable argsort of the class).
 *   u [n] int64 ascending unique row ids in [0, R);  slot_of, last_seen int32 [R];  code int8 [R];  kthr int8 [T];
 *   toff int64 [T] ascending table offsets;  u_next / n_next (host arrays): up to 8 ascending look-ahead id lists
 *   ttl != 0: admit = !hit && last_seen[row] > s, else admit = !hit && in_next;  use_admit != 0: `admit` is an input
 *   (the reference's second classify() after un-admissions, srm2/elara.py:256);  want_T: the planner's st_mode == 'T'
 * Outputs: sl int32 [n], in_next / admit bool bytes [n], c int8 [n] (code of each row), cls int8 [n], counts int64 [11]
 * (classes 0..9; [10] = row ids outside [0, R), classified as C_S without reading anything), order int64 [n].
 */
size_t srm2_plan_scratch_bytes(int64_t n);   /* n = rows of srm2_plan_classify, or dynamic slots of srm2_plan_evict_candidates */
int srm2_plan_classify(const int64_t* u, int64_t n, int64_t R, const int32_t* slot_of, const int32_t* last_seen, const int8_t* code,
                       const int8_t* kthr, const int64_t* toff, int64_t T, const int64_t* const* u_next /* host */,
                       const int64_t* n_next /* host */, int64_t n_lists, int64_t s, int64_t K, int ttl, int want_T, int use_admit,
                       int32_t* sl, uint8_t* in_next, uint8_t* admit, int8_t* c, int8_t* cls, int64_t* counts, int64_t* order,
                       void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* Eviction candidates of a step.  Replaces, inside `ELARAPlanner.plan`, srm2/elara.py:220-228 and :245-246.
 *   protect [C] bool bytes = pinned | (pool slots of the rows in the look-ahead lists);
 *   exp [nd] = !protect[dyn_slots[i]] (ttl != 0: && last_seen[slot_row[dyn_slots[i]]] <= s);
 *   parted [nd] int64 = the dynamic slots, expired ones first, order kept inside both groups; *n_exp (device int64) = their
 *   number: ev_slot = parted[:n_exp], keep_dyn = parted[n_exp:].
 * pinned [C] bool bytes, dyn_slots [nd] int64, slot_row [C] int64; indices out of range are skipped, not read. */
int srm2_plan_evict_candidates(const int64_t* const* u_next /* host */, const int64_t* n_next /* host */, int64_t n_lists,
                               const int32_t* slot_of, int64_t R, const uint8_t* pinned, int64_t C, const int64_t* dyn_slots,
                               int64_t nd, const int64_t* slot_row, const int32_t* last_seen, int64_t s, int ttl,
                               uint8_t* protect, uint8_t* exp, int64_t* n_exp, int64_t* parted, void* scratch, size_t scratch_bytes,
                               srm2_stream_t stream);

/* Packed eviction outputs and host work lists of a plan.  Replaces, inside `ELARAPlanner.plan`, srm2/elara.py:389-407
 * (two stable argsorts, the gathers behind them, loc lookups and the concatenation for the single device-to-host copy).
 *   inputs: ev_slot [nev] int64 and the outputs of srm2_dir_a for them: rep [nev] bool bytes, evf_slots [nev], evl_ids
 *   [nev,K], ev_dyn [nev] int64;  loc int32 [n_loc];  F_row [nF], S_row [nS] int64;  nFa = admitted rows at the head of F_row;
 *   c_slots [nc], a_ids [na] int64 (srm2_dir_b);  L_ids int32 [nL,K] (srm2_dir_a);  mat_top, log_top, live: device int64.
 *   outputs: evM_slot [nev] = ev_slot, rows going to M first;  evl_src [nev*K] = rows of the resident-history matrix, valid
 *   entries first;  flat = S_slot [nS] | F_slot [nF] | L_ids [nL*K] | A_ids [na] | W_slot [nc + nF - nFa + nev] |
 *   EVL_ids [nev*K] | tops [4] = (mat_top, log_top, live, number of rows going back to L), all int64.
 */
size_t srm2_plan_pack_scratch_bytes(int64_t nev, int64_t K);
int srm2_plan_pack(const int64_t* ev_slot, const uint8_t* rep, const int64_t* evf_slots, const int64_t* evl_ids, const int64_t* ev_dyn,
                   int64_t nev, int64_t K, const int32_t* loc, int64_t n_loc, const int64_t* F_row, int64_t nF, int64_t nFa,
                   const int64_t* S_row, int64_t nS, const int64_t* c_slots, int64_t nc, const int32_t* L_ids, int64_t nL,
                   const int64_t* a_ids, int64_t na, const int64_t* mat_top, const int64_t* log_top, const int64_t* live,
                   int64_t* evM_slot, int64_t* evl_src, int64_t* flat, void* scratch, size_t scratch_bytes, srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Pull exchange with sums prepared at the source (no counterpart in the reference).  In the pull form every lookup's
 * gradient row crosses NVLink on its own, although most lookups belong to rows that many lookups of the same rank name,
 * and the owner's run-sum kernel waits an NVLink round trip for each.  The order of summation (runs of ten consecutive
 * lookups of a row, each summed from +0) allows this much: the LEADING lookups of a run that come from one rank can be
 * added up by that rank — same values, same order, same start, hence the same bits — and travel as one row.  (Lookups
 * further back in a run continue a sum that other ranks' rows opened and must be added one by one by the owner.)  With
 * Zipf(1.1) lookups this more than halves the rows that cross.  The source stores what it prepared — sums and the
 * remaining single rows alike — into the owner's memory, so the owner's run-sum kernel reads local memory only.
 *   owner, after srm2_reduce_adam_index(..., SRM2_INDEX_DESCRIPTORS) of a step, same n / D / max_unique / scratch:
 *     srm2_presum_request   per run: two or more leading lookups from one other rank s -> a request {m, positions[10]} in
 *                           region `rank` of rank s's request buffer (peer store), the run's first lookup renamed to the
 *                           entry of region s of this rank's buffer of sums, the others marked as taken; then every
 *                           lookup of another rank that is left -> a request for that one row, renamed the same way.
 *                           A lookup that finds its region full (cap entries per owner and source) stays as it is and is
 *                           read from its source by the run-sum kernel.  The counts go to every source's count array,
 *                           then the barrier (ticket != 0).  n < 2^23.
 *   source, when the step's gradients are in place:
 *     srm2_presum_rows_f32  sums every requested group from `grad` (this rank's [n, D] gradient rows) and stores it into
 *                           entry idx of peer_out[o] = region `rank` of owner o's buffer of sums [cap][D] (peer store);
 *                           its last CTA goes through the barrier (ticket != 0).  A position >= n sets bit 3 (value 8)
 *                           of *err.
 *   owner: srm2_reduce_adam_apply_pull_f32 = srm2_reduce_adam_apply_f32 in pull form with
 *                           peer_out[s] = region s of this rank's buffer of sums (host array of device pointers; NULL:
 *                           no prepared sums in this step) and err = the status word of the exchange (or NULL): when it
 *                           is non-zero at the start of the kernel the step is not applied (a rank that missed a barrier
 *                           must not consume half-written sums; the word is sticky).
 * Both barriers are srm2_peer_barrier's (bounded wait, bit 1 of *err); they need ticket arrays of their own — two further
 * sets of 16 uint64 per rank — because they run on other streams than the exchange's barriers.  All members are 8 bytes wide.
 */
typedef struct srm2_presum {
  int64_t world, rank;
  int64_t cap;                 /* request entries per (source, owner) pair and step, < 2^23 */
  int64_t timeout_ns;
  uint32_t* err;
  void* const* peer_tickets;   /* (host) [world] or NULL */
  uint64_t ticket;             /* 0: no barrier (all ranks' buffers on one device and the calls made in order) */
  /* srm2_presum_request */
  void* const* peer_req;       /* (host) [world]: rank s's request buffer of this step, uint32 [world][cap][12] */
  void* const* peer_req_n;     /* (host) [world]: rank s's request counts of this step, uint32 [world] */
  uint32_t* req_count;         /* [32] counters of this rank for this step, zero before the first call (left zero) */
  /* srm2_presum_rows_f32 */
  const void* req;             /* this rank's request buffer of this step */
  const uint32_t* req_n;       /* this rank's request counts of this step */
  void* const* peer_out;       /* (host) [world]: region `rank` of rank o's buffer of sums of this step, float [cap][D] */
  uint32_t* done;              /* one uint32, zero before the first call (left zero) */
} srm2_presum;
int srm2_presum_request(int64_t n, const int64_t* n_dev, int64_t D, int64_t max_unique, void* scratch, size_t scratch_bytes,
                        const srm2_presum* ps /* host */, srm2_stream_t stream);
int srm2_presum_rows_f32(const float* grad, int64_t n, int64_t D, const srm2_presum* ps /* host */, srm2_stream_t stream);
int srm2_reduce_adam_apply_pull_f32(float* pool, const int64_t* slots, const float* const* peer_grad /* host */,
                                    const float* const* peer_out /* host or NULL */, const uint32_t* err /* or NULL */, int64_t world,
                                    int64_t n, const int64_t* n_dev, int64_t D, int64_t n_unique, const int64_t* n_unique_dev,
                                    int64_t max_unique, const float sc[8] /* host */, void* scratch, size_t scratch_bytes,
                                    srm2_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * A window of K steps as a pipeline of stages on five streams (seven at world > 1), enqueued by one call (no counterpart in the reference;
 * the reference's driver is a Python loop).  It issues exactly the calls documented above, in this order per
 * iteration k — sums(k), descriptors(k+1), sort(k+2), dedup(k+3), exchange(k+4), plan(k+5) — with CUDA events between:
 *   plan (world > 1)      srm2_route_plan                                                  on streams[6]
 *   exchange (world > 1)  srm2_route_publish_barrier, [copy of the step's gradients into its slot],
 *                         srm2_route_dispatch_ids with the barrier in its last CTA         on streams[0]
 *   dedup                 srm2_unique_inverse_nd_i64                                       on streams[1]
 *   sort                  srm2_reduce_adam_index(SRM2_INDEX_SORT)                          on streams[2]
 *   descriptors           srm2_reduce_adam_index(SRM2_INDEX_DESCRIPTORS)                   on streams[3]
 *   sums                  srm2_reduce_adam_apply_f32 (local rows, or peer_grad at world>1) on streams[4], the caller's
 * With presum_cap > 0 the descriptors stage ends with srm2_presum_request, a further stage on streams[5] —
 * srm2_presum_rows_f32(k + 1), which needs that step's gradients but not the table — runs beside sums(k), and the sums
 * stage is srm2_reduce_adam_apply_pull_f32.
 * A host loop that makes these calls itself gives the same result; this entry point exists because at ~20 launches per
 * step the host, not the GPU, bounds such a loop.  All members are 8 bytes wide.  Pointers marked (host) are host
 * arrays; everything else is device memory.  Nothing is allocated or synchronised; the call returns when the window is
 * enqueued, every other stream has been joined into streams[4].
 */
typedef struct srm2_staged {
  int64_t K, first_step, n, D, n_rows, cap_u;   /* n: lookups per step (world 1), capacity of a receive buffer (world > 1) */
  double lr, b1, b2, eps;
  float* pool;                                   /* [n_rows, 3, D] */
  int64_t* counts_out;                           /* [K, 2]: unique rows, invalid ids per step */
  const void* const* ids;                        /* (host) [K] int64 [n_k] */
  const void* const* grads;                      /* (host) [K] float [n_k, D] */
  const int64_t* n_k;                            /* (host) [K] lookups of each step; world 1: all equal n */
  int64_t* u[4]; int64_t* inv[4]; void* scr_s[4];/* four buffer sets: unique rows [cap_u], inverse [n], reduce scratch */
  int64_t scr_s_bytes; void* scr_u; int64_t scr_u_bytes;
  void* const* streams;                          /* (host) [5] cudaStream_t; [7] at world > 1 */
  void* const* events;                           /* (host) [112] cudaEvent_t without timing: 16 per stage */
  void* const* stage_events;                     /* (host) [2K] or NULL: recorded around the sums of each step */
  void* const* trace_events;                     /* (host) [K * 14] or NULL: cudaEvent_t with timing, (begin, end) of exchange,
                                                    dedup, sort, descriptors (requests included), sums, requests, prepared
                                                    sums of every step, step-major (diagnostics) */
  /* world > 1 (pull exchange); ignored at world 1 */
  int64_t world, rank, cap, n_recv_bufs, n_slots, timeout_ns;
  void* route_scr; int64_t route_scr_bytes; int64_t* counts; uint32_t* err; int64_t* n_recv;   /* two route scratch sets of
                                                    route_scr_bytes each, counts [2, world], n_recv [8] */
  int64_t* const* cmat;                          /* (host) [n_recv_bufs] this rank's count matrices */
  int64_t* const* recv_lid;                      /* (host) [n_recv_bufs] this rank's receive buffers (ids) */
  uint32_t* const* recv_src;                     /* (host) [n_recv_bufs] ... (codes) */
  void* const* peer_cmat; void* const* peer_lid; void* const* peer_src;   /* (host) [n_recv_bufs * world] */
  float* const* slot;                            /* (host) [n_slots] this rank's gradient slots */
  const float* const* peer_slot;                 /* (host) [n_slots * world] */
  void* const* peer_tickets;                     /* (host) [world] */
  int64_t* ticket;                               /* (host) in/out: last ticket used */
  /* world > 1, optional: sums prepared at the source (srm2_presum_*); presum_cap == 0 leaves them out */
  int64_t presum_cap;                            /* request entries per (source, owner) pair */
  void* const* peer_req; void* const* peer_req_n;/* (host) [n_slots * world] every rank's request buffers / count arrays */
  const void* const* req;                        /* (host) [n_slots] this rank's request buffers */
  const uint32_t* const* req_n;                  /* (host) [n_slots] this rank's count arrays */
  uint32_t* req_count;                           /* [n_slots][32] counters, zero before the first call */
  void* const* peer_push;                        /* (host) [3 * world] region `rank` of every rank's buffers of sums, by step mod 3 */
  const float* const* peer_out;                  /* (host) [3 * world] the regions of this rank's own buffers of sums */
  void* const* peer_tickets_req; void* const* peer_tickets_sum;   /* (host) [world] each: ticket arrays of the two barriers */
  uint32_t* presum_done;                         /* one zero uint32 */
} srm2_staged;
int srm2_staged_steps(const srm2_staged* a /* host */);

#ifdef __cplusplus
}
#endif
#endif /* SRM2_B200_H */
