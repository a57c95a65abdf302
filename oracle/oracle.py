"""NumPy front-end of the CPU oracle (oracle/srm2_oracle.c) and loader of the compiled reference.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline legs of
bench.py.  The shipped package never imports this module.

All functions take and return NumPy arrays; integer/byte results are exact, fp32 results are the
bits the reference produces (each function cites the reference lines it restates in the C file).
"""
import ctypes as C
import importlib.util
import os
import subprocess
import threading
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None

_i64p = np.ctypeslib.ndpointer(np.int64, flags='C_CONTIGUOUS')
_i32p = np.ctypeslib.ndpointer(np.int32, flags='C_CONTIGUOUS')
_f32p = np.ctypeslib.ndpointer(np.float32, flags='C_CONTIGUOUS')
_u8p = np.ctypeslib.ndpointer(np.uint8, flags='C_CONTIGUOUS')


class _Dir(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in ('code', 'loc', 'ent', 'lstep', 'lfree', 'n_lfree', 'log_top', 'mat_top', 'live',
                                          'adm_c0', 'rj', 'pstep', 'kthr', 'toff', 'slot_of', 'slot_row', 'rok')] + \
               [(k, C.c_int64) for k in ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl', 'T')]


def build():
    """Compile oracle/srm2_oracle.c (gcc, seconds)."""
    subprocess.check_call(['make', '-s', '-C', str(HERE)])


def lib():
    global _LIB
    if _LIB is None:
        so = HERE / '_build' / 'liboracle.so'
        if not so.exists() or so.stat().st_mtime < (HERE / 'srm2_oracle.c').stat().st_mtime:
            build()
        L = C.CDLL(str(so))
        L.orc_adam_scalars.argtypes = [C.c_double] * 4 + [C.c_int64, _f32p]
        L.orc_adam_rows.argtypes = [_f32p, _i64p, _f32p, C.c_int64, C.c_int64, _f32p]
        L.orc_adam_rows_range.argtypes = [_f32p, _i64p, _f32p, C.c_int64, C.c_int64, C.c_int64, _f32p]
        L.orc_init_rows.argtypes = [_f32p, _i64p, C.c_int64, C.c_int64, C.c_uint32, C.c_float]
        L.orc_replay_rows.argtypes = [_f32p, _i64p, _f32p, _i64p, _i32p, _i32p, C.c_int64, C.c_int64, C.c_int64,
                                      C.c_uint32, C.c_float, _f32p]
        L.orc_unique_inverse.argtypes = [_i64p, C.c_int64, _i64p, _i64p]
        L.orc_unique_inverse.restype = C.c_int64
        L.orc_segment_reduce.argtypes = [_f32p, _i64p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, _f32p]
        L.orc_segment_reduce_windowed.argtypes = [_f32p, _i64p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, _f32p]
        L.orc_dir_a.argtypes = [C.POINTER(_Dir), _i64p, C.c_int64, _i64p, _i32p, C.c_int64, _i64p, C.c_int64, C.c_int64,
                                _i32p, _i32p, _i64p, _i64p, _i64p, _u8p, _i64p, _i64p, _i64p]
        L.orc_dir_admit.argtypes = [C.POINTER(_Dir), _i64p, _i64p, C.c_int64, C.c_int64, C.c_int64]
        L.orc_dir_b.argtypes = [C.POINTER(_Dir), _i64p, _i64p, C.c_int64, _i64p, _i64p, C.c_int64, C.c_int64, _i64p, _i64p]
        _LIB = L
    return _LIB


# ---------------------------------------------------------------------------------------------
def adam_scalars(lr, b1, b2, eps, step):
    out = np.empty(8, np.float32)
    lib().orc_adam_scalars(lr, b1, b2, eps, int(step), out)
    return out


def adam_rows(state, rows, grad, lr, b1, b2, eps, step, nthreads=1):
    """In-place row-sparse Adam on state [R,3,D]; with nthreads > 1 the rows are split into contiguous
    chunks the way the reference's cpu_adam splits them (rows must then be distinct)."""
    n, D = rows.shape[0], state.shape[2]
    sc = adam_scalars(lr, b1, b2, eps, step)
    rows = np.ascontiguousarray(rows, np.int64)
    if nthreads <= 1 or n < 256:
        lib().orc_adam_rows(state, rows, grad, n, D, sc)
        return
    chunk = (n + nthreads - 1) // nthreads
    th = []
    for t in range(nthreads):
        lo, hi = t * chunk, min(n, (t + 1) * chunk)
        if lo >= hi:
            break
        th.append(threading.Thread(target=lib().orc_adam_rows_range, args=(state, rows, grad, lo, hi, D, sc)))
        th[-1].start()
    for t in th:
        t.join()


def seed_u32(seed):
    return int(seed) & 0xFFFFFFFF


def init_rows(rows, D, seed, bound):
    rows = np.ascontiguousarray(rows, np.int64)
    out = np.empty((rows.shape[0], 3, D), np.float32)
    lib().orc_init_rows(out, rows, rows.shape[0], D, seed_u32(seed), np.float32(bound))
    return out


def scalar_table(lr, b1, b2, eps, max_step):
    """[max_step+1, 8]; row 0 zeros (srm2/gpu_ops.py:82-88)."""
    t = np.zeros((max_step + 1, 8), np.float32)
    for s in range(1, max_step + 1):
        t[s] = adam_scalars(lr, b1, b2, eps, s)
    return t


def replay_rows(rows, logs, offs, steps, cnt, D, K, seed, bound, table):
    rows = np.ascontiguousarray(rows, np.int64)
    n = rows.shape[0]
    out = np.empty((n, 3, D), np.float32)
    logs = np.ascontiguousarray(logs, np.float32).reshape(-1)
    if logs.size == 0:
        logs = np.zeros(1, np.float32)
    lib().orc_replay_rows(out, rows, logs, np.ascontiguousarray(offs, np.int64), np.ascontiguousarray(steps, np.int32).reshape(-1),
                          np.ascontiguousarray(cnt, np.int32), n, D, K, seed_u32(seed), np.float32(bound),
                          np.ascontiguousarray(table, np.float32).reshape(-1))
    return out


def unique_inverse(ids):
    ids = np.ascontiguousarray(ids, np.int64)
    n = ids.shape[0]
    u = np.empty(max(n, 1), np.int64)
    inv = np.empty(max(n, 1), np.int64)
    nu = lib().orc_unique_inverse(ids if n else np.zeros(1, np.int64), n, u, inv)
    return u[:nu].copy(), inv[:n].copy()


# runs of this many lookups are summed first (see orc_segment_reduce); <= 0: one left-to-right sum
SEGMENT_CHUNK = 10


# inputs of at most this many lookups follow the windowed order (see orc_segment_reduce_windowed)
SEGMENT_SMALL_N = 3072
SEGMENT_WINDOW = 32


def segment_reduce(grad, inv, n_unique, chunk=None, window=None):
    """chunk/window None: the order PyTorch's CUDA operator uses for an input of this size."""
    grad = np.ascontiguousarray(grad, np.float32)
    n, D = grad.shape
    out = np.empty((n_unique, D), np.float32)
    if window is None and chunk is None and n <= SEGMENT_SMALL_N:
        window = SEGMENT_WINDOW
    if window:
        lib().orc_segment_reduce_windowed(grad.reshape(-1) if n else np.zeros(1, np.float32),
                                          np.ascontiguousarray(inv, np.int64) if n else np.zeros(1, np.int64), n, D, n_unique,
                                          window, out.reshape(-1) if n_unique else np.zeros(1, np.float32))
        return out
    ck = SEGMENT_CHUNK if chunk is None else chunk
    lib().orc_segment_reduce(grad.reshape(-1) if n else np.zeros(1, np.float32), np.ascontiguousarray(inv, np.int64) if n else np.zeros(1, np.int64),
                             n, D, n_unique, ck, out.reshape(-1) if n_unique else np.zeros(1, np.float32))
    return out


# ---------------------------------------------------------------------------------------------
DIR_FIELDS = ('code', 'loc', 'ent', 'lstep', 'lfree', 'n_lfree', 'log_top', 'mat_top', 'live', 'adm_c0', 'rj', 'pstep',
              'kthr', 'toff', 'slot_of', 'slot_row', 'rok')
DIR_DTYPES = dict(code=np.int8, loc=np.int32, ent=np.int32, lstep=np.int32, lfree=np.int32, n_lfree=np.int64, log_top=np.int64,
                  mat_top=np.int64, live=np.int64, adm_c0=np.int8, rj=np.int8, pstep=np.int32, kthr=np.int8, toff=np.int64,
                  slot_of=np.int32, slot_row=np.int64, rok=np.int8)


class Directory:
    """State directory on NumPy arrays (srm2/elara.py:117-149); st: dict name -> array, pv: dict of ints
    R, K, Lcap, n0, Cdyn, MAT, trash, evl."""

    def __init__(self, st, pv):
        self.st = {k: np.ascontiguousarray(st[k], DIR_DTYPES[k]) for k in DIR_FIELDS}
        self.pv = dict(pv)
        d = _Dir()
        for k in DIR_FIELDS:
            setattr(d, k, self.st[k].ctypes.data)
        for k in ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl'):
            setattr(d, k, int(pv[k]))
        d.T = self.st['toff'].shape[0]
        self._d = d

    def dir_a(self, hs, L_row, L_cnt, ev_slot, s):
        K = self.pv['K']
        hs = np.ascontiguousarray(hs, np.int64); L_row = np.ascontiguousarray(L_row, np.int64)
        L_cnt = np.ascontiguousarray(L_cnt, np.int32); ev_slot = np.ascontiguousarray(ev_slot, np.int64)
        nh, nL, nev = hs.shape[0], L_row.shape[0], ev_slot.shape[0]
        o = dict(L_steps=np.zeros((nL, K), np.int32), L_ids=np.zeros((nL, K), np.int32), hrec_dyn=np.zeros(nh, np.int64),
                 hrec_j=np.zeros(nh, np.int64), ev_row=np.zeros(nev, np.int64), rep=np.zeros(nev, np.uint8),
                 evl_ids=np.zeros((nev, K), np.int64), evf_slots=np.zeros(nev, np.int64), ev_dyn=np.zeros(nev, np.int64))
        lib().orc_dir_a(C.byref(self._d), hs, nh, L_row, L_cnt, nL, ev_slot, nev, int(s),
                        o['L_steps'].reshape(-1), o['L_ids'].reshape(-1), o['hrec_dyn'], o['hrec_j'], o['ev_row'], o['rep'],
                        o['evl_ids'].reshape(-1), o['evf_slots'], o['ev_dyn'])
        return o

    def admit(self, adm_rows, adm_slots, lazy_n, s):
        adm_rows = np.ascontiguousarray(adm_rows, np.int64); adm_slots = np.ascontiguousarray(adm_slots, np.int64)
        lib().orc_dir_admit(C.byref(self._d), adm_rows, adm_slots, adm_rows.shape[0], int(lazy_n), int(s))

    def dir_b(self, a_rows, a_k, c_rows, c_cnt, s):
        a_rows = np.ascontiguousarray(a_rows, np.int64); a_k = np.ascontiguousarray(a_k, np.int64)
        c_rows = np.ascontiguousarray(c_rows, np.int64); c_cnt = np.ascontiguousarray(c_cnt, np.int64)
        a_ids = np.zeros(a_rows.shape[0], np.int64); c_slots = np.zeros(c_rows.shape[0], np.int64)
        lib().orc_dir_b(C.byref(self._d), a_rows, a_k, a_rows.shape[0], c_rows, c_cnt, c_rows.shape[0], int(s), a_ids, c_slots)
        return dict(a_ids=a_ids, c_slots=c_slots)


def dir_comparable(st, pv):
    """The part of a directory state that is defined by the algorithm: everything except the trash
    destinations (loc[R], ent[R*K:], lstep[Lcap], lfree[Lcap], pstep[Cdyn]) and the stale part of the
    free stack above n_lfree (srm2/elara.py:119-123, 148)."""
    R, K, Lcap, Cdyn = pv['R'], pv['K'], pv['Lcap'], pv['Cdyn']
    nf = int(np.asarray(st['n_lfree']).reshape(-1)[0])
    out = {k: np.asarray(st[k]) for k in DIR_FIELDS}
    out['loc'] = out['loc'][:R]; out['ent'] = out['ent'].reshape(-1)[:R * K]; out['lstep'] = out['lstep'][:Lcap]
    out['lfree'] = out['lfree'][:nf]; out['pstep'] = out['pstep'].reshape(-1, K)[:Cdyn]
    return out


# ---------------------------------------------------------------------------------------------
def _cpu_level():
    try:
        flags = open('/proc/cpuinfo').read().split('flags', 1)[1].split('\n', 1)[0].split()
    except Exception:
        return None
    v4 = {'avx512f', 'avx512bw', 'avx512cd', 'avx512dq', 'avx512vl'}
    v3 = {'avx2', 'fma', 'bmi1', 'bmi2', 'movbe', 'f16c'}
    if v4 <= set(flags) and v3 <= set(flags):
        return 'v4'
    if v3 <= set(flags):
        return 'v3'
    return None


def _load_ext(path, name):
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location(name, str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


_REF = {}


def ref_cpu():
    """The reference's srm2_cpu.cpp compiled by oracle/build_ref.py, or None when it was not built or
    this CPU supports neither ISA level."""
    if 'cpu' not in _REF:
        _REF['cpu'] = None
        lv = _cpu_level()
        if os.environ.get('SRM2_REF_LEVEL'):
            lv = os.environ['SRM2_REF_LEVEL']
        if lv:
            p = HERE / '_ref' / f'srm2_cpu_ext_{lv}.so'
            if p.exists():
                _REF['cpu'] = _load_ext(p, f'srm2_cpu_ext_{lv}')
                _REF['cpu_level'] = lv
    return _REF['cpu']


def ref_dir():
    """The reference's elara_dir.cpp compiled by oracle/build_ref.py, or None."""
    if 'dir' not in _REF:
        p = HERE / '_ref' / 'srm2_elara_dir.so'
        _REF['dir'] = _load_ext(p, 'srm2_elara_dir') if p.exists() else None
    return _REF['dir']


# ------------------------------------------------------------------------------------------------------------
# Classification and class partition of ELARAPlanner.plan (srm2/elara.py:214-219, 229-239, 243, 258), NumPy restatement.
C_HIT, C_NADM, C_NAPP, C_NCMP, C_LADM, C_LAPP, C_LCMP, C_FADM, C_FNADM, C_S = range(10)      # srm2/elara.py:32


def plan_classify(u, u_nexts, slot_of, last_seen, code, kthr, toff, s, K, ttl, want_T, admit=None):
    """-> dict(sl, in_next, admit, c, cls, counts[10], order).  `admit` given: classification only (the reference's second
    call of classify() after un-admissions, srm2/elara.py:256)."""
    u = np.asarray(u, np.int64)
    n = u.shape[0]
    sl = slot_of[u]; hit = sl >= 0                                              # :214
    in_next = np.zeros(n, bool)
    for un in u_nexts:                                                          # :216-218
        j = np.minimum(np.searchsorted(un, u), len(un) - 1)
        in_next |= un[j] == u
    if admit is None:
        admit = ~hit & ((last_seen[u] > s) if ttl else in_next)                 # :219
    c = code[u]; thr = kthr[np.searchsorted(toff, u, side='right') - 1]         # :229, table_of :167-168
    isN = c == 0; isL = (c >= 1) & (c <= K); app = c < thr                      # :230
    wantT = np.full(n, bool(want_T))
    cls = np.full(n, C_S, np.int8)                                              # :235-239
    cls = np.where(~isN & ~isL & (admit | wantT), np.where(admit, C_FADM, C_FNADM), cls)
    cls = np.where(isL, np.where(admit, C_LADM, np.where(app, C_LAPP, C_LCMP)), cls)
    cls = np.where(isN, np.where(admit, C_NADM, np.where(app, C_NAPP, C_NCMP)), cls)
    cls = np.where(hit, C_HIT, cls).astype(np.int8)
    counts = np.bincount(cls.astype(np.int64), minlength=10).astype(np.int64)   # :243
    order = np.argsort(cls, kind='stable').astype(np.int64)                     # :258
    return dict(sl=sl.astype(np.int32), in_next=in_next, admit=admit, c=c.astype(np.int8), cls=cls, counts=counts, order=order)


def plan_positions(r):
    """hit_pos, N_pos, L_pos, F_pos, S_pos as the reference slices them out of `order` (srm2/elara.py:259-266)."""
    b = np.concatenate([[0], np.cumsum(r['counts'])])
    rng = lambda lo, hi: r['order'][b[lo]:b[hi + 1]]
    return dict(hit_pos=rng(C_HIT, C_HIT), N_pos=rng(C_NADM, C_NCMP), L_pos=rng(C_LADM, C_LCMP), F_pos=rng(C_FADM, C_FNADM), S_pos=rng(C_S, C_S))


def plan_evict_candidates(u_nexts, slot_of, pinned, dyn_slots, slot_row, last_seen, s, ttl):
    """Eviction candidates of a step (srm2/elara.py:220-228, 245-246): slots named by the look-ahead lists are protected;
    a dynamic slot expires when it is not protected (TTL mode: and its row's last_seen <= s); the dynamic slots are split,
    keeping their order, into the expired ones (ev_slot) and the rest (keep_dyn).
    -> dict(protect bool [C], exp bool [len(dyn_slots)], n_exp, ev_slot, keep_dyn)."""
    protect = pinned.copy()                                                        # :220
    for un in u_nexts:                                                             # :221-223
        sn = slot_of[un].astype(np.int64)
        protect[sn[sn >= 0]] = True
    dl = np.asarray(dyn_slots, np.int64)
    exp = ~protect[dl]                                                             # :226
    if ttl:
        exp &= last_seen[slot_row[dl]] <= s                                        # :227-228
    o = np.argsort(~exp, kind='stable')                                            # :245
    n_exp = int(exp.sum())
    return dict(protect=protect, exp=exp, n_exp=n_exp, ev_slot=dl[o[:n_exp]], keep_dyn=dl[o[n_exp:]])


def plan_pack(ev_slot, rep, evf_slots, evl_ids, ev_dyn, K, loc, F_row, S_row, nFa, c_slots, L_ids, a_ids, tops3):
    """Packed eviction outputs and host work lists of a plan (srm2/elara.py:389-407).
    -> dict(evM_slot, evl_src, S_slot, F_slot, L_ids, A_ids, W_slot, EVL_ids, tops[4])."""
    nev = len(ev_slot)
    if nev:
        om = np.argsort(rep.astype(np.int8), kind='stable')                     # rows going to M first (:393-394)
        evM_slot = ev_slot[om]; evf = evf_slots[om]
        flat = evl_ids.reshape(-1)
        ol = np.argsort((flat < 0).astype(np.int8), kind='stable')              # valid history entries first (:395-397)
        evl_src = (ev_dyn[:, None] * K + np.arange(K)[None, :]).reshape(-1)[ol]
        evl = flat[ol]
    else:
        evM_slot = ev_slot; evf = evf_slots; evl_src = np.zeros(0, np.int64); evl = evl_ids.reshape(-1)
    F_slot = loc[F_row].astype(np.int64); S_slot = loc[S_row].astype(np.int64)  # :401
    W_slot = np.concatenate([c_slots, F_slot[nFa:], evf])                       # :402
    tops = np.concatenate([np.asarray(tops3, np.int64), [int(rep.sum())]])      # :403
    return dict(evM_slot=evM_slot, evl_src=evl_src, S_slot=S_slot, F_slot=F_slot, L_ids=L_ids.reshape(-1).astype(np.int64),
                A_ids=a_ids.astype(np.int64), W_slot=W_slot, EVL_ids=evl.astype(np.int64), tops=tops)
