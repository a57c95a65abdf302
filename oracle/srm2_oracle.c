/*
 * CPU oracle for the sparse-optimizer hot path of ELARA (srm2).
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain sequential C, the algorithms of the
 * reference implementation so that the CUDA kernels can be checked bit for bit.  Nothing in the
 * shipped library may link, load or call it; only the test-suite, the smoke check and the CPU
 * baseline leg of the benchmark do.
 *
 * Every function names the reference lines it follows (paths relative to the reference project).
 * Floating-point code is compiled with -ffp-contract=off -fno-fast-math: every operation is a
 * separately rounded IEEE fp32 operation, exactly as the reference demands.
 *
 * Parity pins (see tests/test_oracle_golden.py):
 *   adam, scalars      : the reference's own cpu_adam / adam_scalars (built from its C++ source)
 *   init, replay       : the reference's Triton kernels run under the Triton CPU interpreter
 *   directory a/b      : the reference's elara_dir.cpp driven by its own ELARAPlanner on CPU tensors
 *   unique             : integer only (torch.unique on CPU)
 *   segment-reduce     : third-party arithmetic (PyTorch aten::embedding_dense_backward, CUDA build,
 *                        torch==2.11.0); pinned by vectors produced by that operator on a B200.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* zero-filled scratch of at least one element */
#define ORC_NEW(type, n) ((type*)calloc((size_t)((n) > 0 ? (n) : 1), sizeof(type)))

/* ------------------------------------------------------------------------------------------- */
/* Adam scalars: srm2/csrc/srm2_cpu.cpp:13-20 (make_scalars) and :255-257 (adam_scalars export). */
/* Each of the 8 values is evaluated in double precision and rounded to float exactly once.      */
void orc_adam_scalars(double lr, double b1, double b2, double eps, int64_t step, float out[8]) {
  out[0] = (float)lr;
  out[1] = (float)b1;
  out[2] = (float)(1.0 - b1);
  out[3] = (float)b2;
  out[4] = (float)(1.0 - b2);
  out[5] = (float)(1.0 - pow(b1, (double)step));
  out[6] = (float)(1.0 - pow(b2, (double)step));
  out[7] = (float)eps;
}

/* One Adam step on one element; srm2/csrc/srm2_cpu.cpp:26-32 == srm2/ops.py:50-56.              */
static inline void adam_elem(float* w, float* m, float* v, float g, const float* s) {
  const float lr = s[0], b1 = s[1], omb1 = s[2], b2 = s[3], omb2 = s[4], bc1 = s[5], bc2 = s[6], eps = s[7];
  float mj = b1 * *m; float t1 = omb1 * g; mj = mj + t1;
  float vj = b2 * *v; float t2 = omb2 * g; t2 = t2 * g; vj = vj + t2;
  float mh = mj / bc1; float vh = vj / bc2;
  float den = sqrtf(vh); den = den + eps;
  float num = lr * mh; float up = num / den;
  *w = *w - up; *m = mj; *v = vj;
}

/* Row-sparse Adam on interleaved state [R,3,D]; srm2/csrc/srm2_cpu.cpp:36-56 (cpu_adam), serial. */
void orc_adam_rows(float* state, const int64_t* rows, const float* grad, int64_t n, int64_t D, const float sc[8]) {
  for (int64_t i = 0; i < n; ++i) {
    float* base = state + rows[i] * 3 * D;
    const float* g = grad + i * D;
    for (int64_t j = 0; j < D; ++j) adam_elem(base + j, base + D + j, base + 2 * D + j, g[j], sc);
  }
}

/* The same, split over a contiguous range so that a caller may run several threads of it the    */
/* way cpu_adam does (srm2_cpu.cpp:49-55: contiguous chunks of ceil(n / nthreads) rows).          */
void orc_adam_rows_range(float* state, const int64_t* rows, const float* grad, int64_t lo, int64_t hi, int64_t D,
                         const float sc[8]) {
  for (int64_t i = lo; i < hi; ++i) {
    float* base = state + rows[i] * 3 * D;
    const float* g = grad + i * D;
    for (int64_t j = 0; j < D; ++j) adam_elem(base + j, base + D + j, base + 2 * D + j, g[j], sc);
  }
}

/* ------------------------------------------------------------------------------------------- */
/* murmur3 fmix32; srm2/gpu_ops.py:15-23 (_hash32).                                              */
static inline uint32_t fmix32(uint32_t x) {
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

/* Initial weight of element j of row r; srm2/gpu_ops.py:29-34.                                   */
/* r*D+j and r>>32 are formed in int64 and truncated to uint32; u = (h>>8)*2^-24 is exact;        */
/* u*2-1 is exact (a multiple of 2^-23 in [-1,1)); the product with bound is the only rounding.   */
static inline float init_elem(int64_t r, int64_t D, int64_t j, uint32_t seed, float bound) {
  uint32_t key = (uint32_t)(uint64_t)(r * D + j) ^ fmix32((uint32_t)(uint64_t)(r >> 32) + seed);
  uint32_t h = fmix32(key ^ seed);
  float u = (float)(h >> 8) * (1.0f / 16777216.0f);
  float t = u * 2.0f; t = t - 1.0f;
  return t * bound;
}

/* Counter-hash row initialisation; srm2/gpu_ops.py:26-48 (_init_rows, init_rows). out [n,3,D].  */
void orc_init_rows(float* out, const int64_t* rows, int64_t n, int64_t D, uint32_t seed, float bound) {
  for (int64_t i = 0; i < n; ++i) {
    float* base = out + i * 3 * D;
    for (int64_t j = 0; j < D; ++j) { base[j] = init_elem(rows[i], D, j, seed, bound); base[D + j] = 0.0f; base[2 * D + j] = 0.0f; }
  }
}

/* Exact replay of up to K logged gradients; srm2/gpu_ops.py:51-79 (_replay) and :91-99.          */
/* table: [table_rows, 8] Adam scalars per logical step (row 0 zeros), srm2/gpu_ops.py:82-88.     */
void orc_replay_rows(float* out, const int64_t* rows, const float* logs, const int64_t* offs, const int32_t* steps,
                     const int32_t* cnt, int64_t n, int64_t D, int64_t K, uint32_t seed, float bound,
                     const float* table) {
  for (int64_t i = 0; i < n; ++i) {
    float* base = out + i * 3 * D;
    const int32_t c = cnt[i]; const int64_t o = offs[i];
    for (int64_t j = 0; j < D; ++j) {
      float w = init_elem(rows[i], D, j, seed, bound), m = 0.0f, v = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        if (k < c) {
          const float* sc = table + (int64_t)steps[i * K + k] * 8;
          adam_elem(&w, &m, &v, logs[(o + k) * D + j], sc);
        }
      }
      base[j] = w; base[D + j] = m; base[2 * D + j] = v;
    }
  }
}

/* ------------------------------------------------------------------------------------------- */
/* Dedup; call site srm2/train.py:352: torch.unique(ids, return_inverse=True) -> sorted unique   */
/* values and, per input position, the index of its value in the unique list.  Integer only.     */
typedef struct { int64_t id; int64_t pos; } idpos_t;
static int cmp_idpos(const void* a, const void* b) {
  const idpos_t* x = (const idpos_t*)a; const idpos_t* y = (const idpos_t*)b;
  if (x->id != y->id) return x->id < y->id ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos);
}
/* returns the number of unique ids; uniq must hold n entries, inv n entries.                    */
int64_t orc_unique_inverse(const int64_t* ids, int64_t n, int64_t* uniq, int64_t* inv) {
  if (n == 0) return 0;
  idpos_t* t = ORC_NEW(idpos_t, n);
  for (int64_t i = 0; i < n; ++i) { t[i].id = ids[i]; t[i].pos = i; }
  qsort(t, (size_t)n, sizeof(idpos_t), cmp_idpos);
  int64_t nu = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (i == 0 || t[i].id != t[i - 1].id) uniq[nu++] = t[i].id;
    inv[t[i].pos] = nu - 1;
  }
  free(t);
  return nu;
}

/* Segment-reduce; call site srm2/train.py:429:                                                   */
/*   aten.embedding_dense_backward(grad[n,D], inv[n], n_unique, -1, False) -> [n_unique, D].     */
/* The arithmetic lives in PyTorch (pinned torch==2.11.0), not in the reference tree.  The order  */
/* of the fp32 additions is that operator's, restated here as a two-level sum:                    */
/*   the lookups of one unique row, taken in ascending lookup position, are cut into runs of      */
/*   `chunk` lookups; each run is summed left to right starting from +0; the run sums are then    */
/*   added left to right starting from +0.  chunk <= 0 means one single left-to-right sum         */
/*   starting from the first element (PyTorch's CPU kernel order).                                */
void orc_segment_reduce(const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t n_unique, int64_t chunk,
                        float* out) {
  /* stable counting sort of positions by inv */
  int64_t* start = ORC_NEW(int64_t, n_unique + 1);
  int64_t* order = ORC_NEW(int64_t, n);
  for (int64_t p = 0; p < n; ++p) start[inv[p] + 1]++;
  for (int64_t j = 0; j < n_unique; ++j) start[j + 1] += start[j];
  int64_t* fill = ORC_NEW(int64_t, n_unique);
  memcpy(fill, start, (size_t)n_unique * sizeof(int64_t));
  for (int64_t p = 0; p < n; ++p) order[fill[inv[p]]++] = p;
  for (int64_t j = 0; j < n_unique; ++j) {
    const int64_t a = start[j], b = start[j + 1];
    for (int64_t d = 0; d < D; ++d) {
      if (b == a) { out[j * D + d] = 0.0f; continue; }
      if (chunk <= 0) {
        float acc = grad[order[a] * D + d];
        for (int64_t q = a + 1; q < b; ++q) acc = acc + grad[order[q] * D + d];
        out[j * D + d] = acc;
      } else {
        float tot = 0.0f;
        for (int64_t c0 = a; c0 < b; c0 += chunk) {
          const int64_t c1 = c0 + chunk < b ? c0 + chunk : b;
          float part = 0.0f;
          for (int64_t q = c0; q < c1; ++q) part = part + grad[order[q] * D + d];
          tot = tot + part;
        }
        out[j * D + d] = tot;
      }
    }
  }
  free(start); free(order); free(fill);
}

/* Small-input order of the same operator (inputs of at most a few thousand lookups take a different  */
/* kernel inside PyTorch): the lookups are walked in windows of `window` consecutive positions; inside */
/* a window the lookups of one unique row are summed left to right starting from the first of them,   */
/* and that window sum is then added to the output row, which starts at +0.                           */
void orc_segment_reduce_windowed(const float* grad, const int64_t* inv, int64_t n, int64_t D, int64_t n_unique,
                                 int64_t window, float* out) {
  for (int64_t t = 0; t < n_unique * D; ++t) out[t] = 0.0f;
  uint8_t* done = ORC_NEW(uint8_t, window);
  for (int64_t w0 = 0; w0 < n; w0 += window) {
    const int64_t w1 = w0 + window < n ? w0 + window : n;
    memset(done, 0, (size_t)window);
    for (int64_t p = w0; p < w1; ++p) {
      if (done[p - w0]) continue;
      const int64_t j = inv[p];
      for (int64_t d = 0; d < D; ++d) {
        float acc = grad[p * D + d];
        for (int64_t q = p + 1; q < w1; ++q) if (inv[q] == j) acc = acc + grad[q * D + d];
        out[j * D + d] = out[j * D + d] + acc;
      }
      for (int64_t q = p + 1; q < w1; ++q) if (inv[q] == j) done[q - w0] = 1;
    }
  }
  free(done);
}

/* ------------------------------------------------------------------------------------------- */
/* State directory; state layout srm2/csrc/elara_dir.cpp:8-11, built at srm2/elara.py:117-149.   */
typedef struct {
  int8_t* code;        /* [R]            0 = I, 1..K = L_c, MAT = M                         */
  int32_t* loc;        /* [R+1]          MAT slot, last = trash                             */
  int32_t* ent;        /* [(R+1)*K]      log-entry ids, last row = trash                    */
  int32_t* lstep;      /* [Lcap+1]       logical step per log entry, last = trash           */
  int32_t* lfree;      /* [Lcap+1]       free stack of log ids, last = trash                */
  int64_t* n_lfree;    /* [1] */
  int64_t* log_top;    /* [1] */
  int64_t* mat_top;    /* [1] */
  int64_t* live;       /* [1] */
  int8_t* adm_c0;      /* [C] */
  int8_t* rj;          /* [C] */
  int32_t* pstep;      /* [Cdyn+1, K]    last row = trash                                   */
  const int8_t* kthr;  /* [T] */
  const int64_t* toff; /* [T] ascending table offsets */
  int32_t* slot_of;    /* [R] */
  int64_t* slot_row;   /* [C] */
  int8_t* rok;         /* [C] */
  int64_t R, K, Lcap, n0, Cdyn, MAT, trash, evl, T;
} orc_dir_t;

/* srm2/csrc/elara_dir.cpp:46-48: searchsorted(toff, row, right=True) - 1.                        */
static int64_t table_of(const orc_dir_t* s, int64_t row) {
  int64_t lo = 0, hi = s->T;
  while (lo < hi) { int64_t mid = (lo + hi) / 2; if (s->toff[mid] <= row) lo = mid + 1; else hi = mid; }
  return lo - 1;
}

/* srm2/csrc/elara_dir.cpp:13-21 (alloc_logs): ids for the valid lanes, free stack first (top    */
/* downwards), then the bump pointer; counters updated after all ids are formed.                  */
static void alloc_logs(orc_dir_t* s, const uint8_t* valid, int64_t m, int64_t* ids) {
  const int64_t nf = *s->n_lfree, top = *s->log_top;
  int64_t rank = -1;
  for (int64_t t = 0; t < m; ++t) {
    if (valid[t]) ++rank;
    if (rank < nf) { int64_t ix = nf - 1 - rank; if (ix < 0) ix = 0; ids[t] = s->lfree[ix]; }
    else ids[t] = top + rank - nf;
  }
  const int64_t k = rank + 1, used = k < nf ? k : nf;
  *s->log_top += k - used; *s->n_lfree -= used; *s->live += k;
}

/* srm2/csrc/elara_dir.cpp:23-34 (free_logs): push the first cnt[i] live entries of rows[i].      */
static void free_logs(orc_dir_t* s, const int64_t* rows, const int64_t* cnt, int64_t n) {
  if (n == 0) return;
  const int64_t K = s->K, nf = *s->n_lfree;
  int64_t rank = -1;
  for (int64_t i = 0; i < n; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t pos = rows[i] * K + k; const int32_t e = s->ent[pos];
      const int valid = (k < cnt[i]) && (e >= 0);
      if (valid) { ++rank; s->lfree[nf + rank] = e; } else s->lfree[s->Lcap] = e;
    }
  for (int64_t i = 0; i < n; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t pos = rows[i] * K + k; const int32_t e = s->ent[pos];
      const int valid = (k < cnt[i]) && (e >= 0);
      s->ent[valid ? pos : s->R * K] = -1;
    }
  *s->n_lfree += rank + 1; *s->live -= rank + 1;
}

/* srm2/csrc/elara_dir.cpp:36-44 (alloc_mat): rows without a MAT slot (and inside mask) get       */
/* consecutive slots in order.                                                                    */
static void alloc_mat(orc_dir_t* s, const int64_t* rows, const uint8_t* mask, int64_t n, int64_t* sl) {
  const int64_t top = *s->mat_top; int64_t rank = -1;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t cur = s->loc[rows[i]];
    const int nw = cur < 0 && (mask == NULL || mask[i]);
    if (nw) ++rank;
    sl[i] = nw ? top + rank : cur;
  }
  for (int64_t i = 0; i < n; ++i) s->loc[rows[i]] = (int32_t)sl[i];
  *s->mat_top += rank + 1;
}

/* Call A; srm2/csrc/elara_dir.cpp:50-96 (elara_dir_a), twin srm2/elara.py:285-343.               */
void orc_dir_a(orc_dir_t* s, const int64_t* hs, int64_t nh, const int64_t* L_row, const int32_t* L_cnt, int64_t nL,
               const int64_t* ev_slot, int64_t nev, int64_t step,
               int32_t* L_steps, int32_t* L_ids, int64_t* hrec_dyn, int64_t* hrec_j, int64_t* ev_row, uint8_t* rep,
               int64_t* evl_ids, int64_t* evf_slots, int64_t* ev_dyn) {
  const int64_t K = s->K;
  /* replay inputs (:57-59) */
  for (int64_t i = 0; i < nL; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const int32_t e = s->ent[L_row[i] * K + k];
      L_steps[i * K + k] = e >= 0 ? s->lstep[e] : 0;
      L_ids[i * K + k] = k < L_cnt[i] ? e : -1;
    }
  /* hits (:61-71); hs holds distinct slots, every read precedes every write */
  for (int64_t i = 0; i < nh; ++i) {
    const int64_t sl = hs[i];
    const int dyn = sl >= s->n0; const int64_t c0 = s->adm_c0[sl], j = s->rj[sl]; const int ok = s->rok[sl] != 0;
    const int rec = s->evl ? (dyn && ok && (c0 + j) < K) : 0;
    hrec_dyn[i] = rec ? sl - s->n0 : s->Cdyn; hrec_j[i] = rec ? j : 0;
  }
  for (int64_t i = 0; i < nh; ++i) {
    const int64_t sl = hs[i];
    const int dyn = sl >= s->n0; const int64_t j = s->rj[sl]; const int ok = s->rok[sl] != 0;
    const int rec = hrec_dyn[i] != s->Cdyn;
    s->pstep[hrec_dyn[i] * K + hrec_j[i]] = (int32_t)step;
    s->rj[sl] = (int8_t)(j + rec);
    s->rok[sl] = (int8_t)(ok && !(dyn && !rec));
  }
  /* evictions (:73-94) */
  int64_t* c0v = ORC_NEW(int64_t, nev);
  int64_t* jv = ORC_NEW(int64_t, nev);
  for (int64_t i = 0; i < nev; ++i) {
    ev_row[i] = s->slot_row[ev_slot[i]]; c0v[i] = s->adm_c0[ev_slot[i]]; jv[i] = s->rj[ev_slot[i]];
    rep[i] = (s->evl && nev) ? ((s->rok[ev_slot[i]] != 0) && (c0v[i] + jv[i] <= (int64_t)s->kthr[table_of(s, ev_row[i])])) : 0;
    ev_dyn[i] = ev_slot[i] - s->n0;
  }
  for (int64_t i = 0; i < nev; ++i) { s->slot_of[ev_row[i]] = -1; s->slot_row[ev_slot[i]] = -1; }
  uint8_t* valid = ORC_NEW(uint8_t, nev * K);
  for (int64_t i = 0; i < nev; ++i) for (int64_t k = 0; k < K; ++k) valid[i * K + k] = rep[i] && k < jv[i];
  alloc_logs(s, valid, nev * K, evl_ids);
  for (int64_t t = 0; t < nev * K; ++t) if (!valid[t]) evl_ids[t] = -1;
  for (int64_t i = 0; i < nev; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t t = i * K + k; const int64_t c0 = c0v[i] > 0 ? c0v[i] : 0;
      const int64_t pos = valid[t] ? ev_row[i] * K + c0 + k : s->R * K;
      s->ent[pos] = (int32_t)evl_ids[t];
    }
  for (int64_t i = 0; i < nev; ++i)
    for (int64_t k = 0; k < K; ++k) {
      const int64_t t = i * K + k;
      s->lstep[valid[t] ? evl_ids[t] : s->Lcap] = s->pstep[ev_dyn[i] * K + k];
    }
  uint8_t* nrep = ORC_NEW(uint8_t, nev);
  for (int64_t i = 0; i < nev; ++i) nrep[i] = !rep[i];
  alloc_mat(s, ev_row, nrep, nev, evf_slots);
  for (int64_t i = 0; i < nev; ++i) if (rep[i]) evf_slots[i] = s->trash;
  if (nev) {
    int64_t* fc = ORC_NEW(int64_t, nev);
    for (int64_t i = 0; i < nev; ++i) fc[i] = rep[i] ? 0 : (c0v[i] > 0 ? c0v[i] : 0);
    free_logs(s, ev_row, fc, nev);
    for (int64_t i = 0; i < nev; ++i) {
      int64_t c = c0v[i] + jv[i]; if (c > 127) c = 127;
      s->code[ev_row[i]] = rep[i] ? (int8_t)c : (int8_t)s->MAT;
    }
    free(fc);
  }
  free(c0v); free(jv); free(valid); free(nrep);
}

/* Pool-slot admissions between the two directory calls; srm2/elara.py:358-366.                   */
/* adm_rows = N_adm || L_adm || F_adm; the first lazy_n come from states I/L.                      */
void orc_dir_admit(orc_dir_t* s, const int64_t* adm_rows, const int64_t* adm_slots, int64_t n_adm, int64_t lazy_n,
                   int64_t step) {
  for (int64_t i = 0; i < n_adm; ++i) {
    const int64_t r = adm_rows[i], sl = adm_slots[i];
    const int lazy = (i < lazy_n) && s->evl;
    s->slot_of[r] = (int32_t)sl; s->slot_row[sl] = r;
    s->adm_c0[sl] = (i < lazy_n) ? s->code[r] : (int8_t)-1;
    s->rj[sl] = (int8_t)lazy; s->rok[sl] = (int8_t)lazy;
    if (lazy) s->pstep[(sl - s->n0) * s->K] = (int32_t)step;
  }
}

/* Call B; srm2/csrc/elara_dir.cpp:98-110 (elara_dir_b), twin srm2/elara.py:380-386.              */
void orc_dir_b(orc_dir_t* s, const int64_t* a_rows, const int64_t* a_k, int64_t na, const int64_t* c_rows,
               const int64_t* c_cnt, int64_t nc, int64_t step, int64_t* a_ids, int64_t* c_slots) {
  const int64_t K = s->K;
  uint8_t* ones = ORC_NEW(uint8_t, na); memset(ones, 1, (size_t)(na > 0 ? na : 1));
  alloc_logs(s, ones, na, a_ids);
  for (int64_t i = 0; i < na; ++i) {
    s->ent[a_rows[i] * K + a_k[i]] = (int32_t)a_ids[i]; s->lstep[a_ids[i]] = (int32_t)step;
    s->code[a_rows[i]] = (int8_t)(a_k[i] + 1);
  }
  alloc_mat(s, c_rows, NULL, nc, c_slots);
  if (nc) {
    free_logs(s, c_rows, c_cnt, nc);
    for (int64_t i = 0; i < nc; ++i) s->code[c_rows[i]] = (int8_t)s->MAT;
  }
  free(ones);
}
