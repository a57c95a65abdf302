"""Planner-side kernels: the classification and class partition of `ELARAPlanner.plan` (reference: srm2/elara.py:209-271).

    r = plan_classify(u, u_nexts, pl.slot_of, pl.last_seen, pl.code, pl.kthr, pl.toff, s, pl.Kmax, pl.dyn == 'ttl', pl.st_mode == 'T')
    sl, hit, admit, c, cls, counts, order = r.sl, r.sl >= 0, r.admit, r.c, r.cls, r.counts, r.order

gives the tensors the reference computes at srm2/elara.py:214-219, 229-239, 243 and 258 in four launches.
"""
import ctypes as C
from types import SimpleNamespace

import torch

from . import _lib, ops

CLASSES = ('HIT', 'NADM', 'NAPP', 'NCMP', 'LADM', 'LAPP', 'LCMP', 'FADM', 'FNADM', 'S')      # srm2/elara.py:32


def plan_classify(u, u_nexts, slot_of, last_seen, code, kthr, toff, s, K, ttl, want_T, admit=None):
    """u: cuda int64 [n] ascending unique rows; u_nexts: list of up to 8 such tensors (the look-ahead window).
    Returns a namespace of cuda tensors: sl int32, in_next bool, admit bool, c int8, cls int8, counts int64 [10] (still on
    the device: the reference reads them with its one host sync), order int64 (stable argsort of cls).
    admit given: classification with that admission mask (the reference's second classify(), srm2/elara.py:256)."""
    if not u.is_cuda:
        raise RuntimeError('u must be a CUDA tensor: this library has no CPU path')
    dev, n = u.device, u.numel()
    if len(u_nexts) > 8:
        raise RuntimeError('at most 8 look-ahead lists')
    for name, t, dt in (('u', u, torch.int64), ('slot_of', slot_of, torch.int32), ('last_seen', last_seen, torch.int32), ('code', code, torch.int8),
                        ('kthr', kthr, torch.int8), ('toff', toff, torch.int64), *[(f'u_nexts[{q}]', t, torch.int64) for q, t in enumerate(u_nexts)]):
        if t.dtype != dt or not t.is_contiguous() or t.device != dev:
            raise RuntimeError(f'{name} must be a contiguous {dt} tensor on the device of u')
    L = _lib.lib()
    sl = torch.empty(n, dtype=torch.int32, device=dev)
    in_next = torch.empty(n, dtype=torch.bool, device=dev)
    if admit is None:
        adm, use = torch.empty(n, dtype=torch.bool, device=dev), 0
    else:
        if admit.dtype != torch.bool or admit.numel() != n or admit.device != dev:
            raise RuntimeError('admit must be a bool tensor [n] on the device of u')
        adm, use = admit.contiguous().clone(), 1
    c = torch.empty(n, dtype=torch.int8, device=dev)
    cls = torch.empty(n, dtype=torch.int8, device=dev)
    counts = torch.empty(11, dtype=torch.int64, device=dev)
    order = torch.empty(n, dtype=torch.int64, device=dev)
    scr = ops._scratch(dev, L.srm2_plan_scratch_bytes(n), 'plan')
    nl = len(u_nexts)
    ptrs = (C.c_void_p * max(nl, 1))(*[t.data_ptr() for t in u_nexts])
    lens = (C.c_int64 * max(nl, 1))(*[t.numel() for t in u_nexts])
    with torch.cuda.device(dev):
        st = L.srm2_plan_classify(u.data_ptr(), n, code.numel(), slot_of.data_ptr(), last_seen.data_ptr(), code.data_ptr(), kthr.data_ptr(),
                                  toff.data_ptr(), toff.numel(), ptrs, lens, nl, int(s), int(K), int(bool(ttl)), int(bool(want_T)), use,
                                  sl.data_ptr(), in_next.data_ptr(), adm.data_ptr(), c.data_ptr(), cls.data_ptr(), counts.data_ptr(),
                                  order.data_ptr(), scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'plan_classify')
    return SimpleNamespace(sl=sl, in_next=in_next, admit=adm, c=c, cls=cls, counts=counts[:10], bad_rows=counts[10:], order=order)


def evict_candidates(u_nexts, slot_of, pinned, dyn_slots, slot_row, last_seen, s, ttl):
    """Eviction candidates of a step (reference: srm2/elara.py:220-228, 245-246).  Returns a namespace of cuda tensors:
    protect bool [C], exp bool [len(dyn_slots)], n_exp int64 [1] (on the device: the reference reads it with the class counts
    in its one host sync), parted int64: ev_slot = parted[:n_exp], keep_dyn = parted[n_exp:]."""
    if not slot_of.is_cuda:
        raise RuntimeError('slot_of must be a CUDA tensor: this library has no CPU path')
    dev = slot_of.device
    if len(u_nexts) > 8:
        raise RuntimeError('at most 8 look-ahead lists')
    for name, t, dt in (('slot_of', slot_of, torch.int32), ('pinned', pinned, torch.bool), ('dyn_slots', dyn_slots, torch.int64),
                        ('slot_row', slot_row, torch.int64), ('last_seen', last_seen, torch.int32),
                        *[(f'u_nexts[{q}]', t, torch.int64) for q, t in enumerate(u_nexts)]):
        if t.dtype != dt or not t.is_contiguous() or t.device != dev:
            raise RuntimeError(f'{name} must be a contiguous {dt} tensor on the device of slot_of')
    L = _lib.lib()
    Cn, nd = pinned.numel(), dyn_slots.numel()
    protect = torch.empty(Cn, dtype=torch.bool, device=dev)
    exp = torch.empty(nd, dtype=torch.bool, device=dev)
    n_exp = torch.empty(1, dtype=torch.int64, device=dev)
    parted = torch.empty(nd, dtype=torch.int64, device=dev)
    scr = ops._scratch(dev, L.srm2_plan_scratch_bytes(nd), 'plan')
    nl = len(u_nexts)
    ptrs = (C.c_void_p * max(nl, 1))(*[t.data_ptr() for t in u_nexts])
    lens = (C.c_int64 * max(nl, 1))(*[t.numel() for t in u_nexts])
    with torch.cuda.device(dev):
        st = L.srm2_plan_evict_candidates(ptrs, lens, nl, slot_of.data_ptr(), slot_of.numel(), pinned.data_ptr(), Cn, dyn_slots.data_ptr(), nd,
                                          slot_row.data_ptr(), last_seen.data_ptr(), int(s), int(bool(ttl)), protect.data_ptr(), exp.data_ptr(),
                                          n_exp.data_ptr(), parted.data_ptr(), scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'plan_evict_candidates')
    return SimpleNamespace(protect=protect, exp=exp, n_exp=n_exp, parted=parted)


def pack(ev_slot, rep, evf_slots, evl_ids, ev_dyn, K, loc, F_row, S_row, nFa, c_slots, L_ids, a_ids, mat_top, log_top, live):
    """Packed eviction outputs and host work lists of a plan (reference: srm2/elara.py:389-407).  Returns a namespace:
    evM_slot, evl_src (cuda int64) and `flat` (cuda int64) with `parts`, the (name, length) list in emission order —
    the reference copies exactly this buffer to the host in its one device-to-host copy and slices it there."""
    dev = loc.device
    if not loc.is_cuda:
        raise RuntimeError('loc must be a CUDA tensor: this library has no CPU path')
    nev, nF, nS, nc, nL, na = ev_slot.numel(), F_row.numel(), S_row.numel(), c_slots.numel(), L_ids.numel() // max(K, 1), a_ids.numel()
    for name, t, dt in (('ev_slot', ev_slot, torch.int64), ('rep', rep, torch.bool), ('evf_slots', evf_slots, torch.int64),
                        ('evl_ids', evl_ids, torch.int64), ('ev_dyn', ev_dyn, torch.int64), ('loc', loc, torch.int32), ('F_row', F_row, torch.int64),
                        ('S_row', S_row, torch.int64), ('c_slots', c_slots, torch.int64), ('L_ids', L_ids, torch.int32), ('a_ids', a_ids, torch.int64),
                        ('mat_top', mat_top, torch.int64), ('log_top', log_top, torch.int64), ('live', live, torch.int64)):
        if t.numel() and (t.dtype != dt or not t.is_contiguous() or t.device != dev):
            raise RuntimeError(f'{name} must be a contiguous {dt} tensor on the device of loc')
    if rep.numel() != nev or evf_slots.numel() != nev or ev_dyn.numel() != nev or evl_ids.numel() != nev * K:
        raise RuntimeError('rep, evf_slots, ev_dyn must be [nev] and evl_ids [nev, K]')
    parts = [('S_slot', nS), ('F_slot', nF), ('L_ids', nL * K), ('A_ids', na), ('W_slot', nc + nF - int(nFa) + nev), ('EVL_ids', nev * K), ('tops', 4)]
    L = _lib.lib()
    evM_slot = torch.empty(nev, dtype=torch.int64, device=dev)
    evl_src = torch.empty(nev * K, dtype=torch.int64, device=dev)
    flat = torch.empty(sum(n for _, n in parts), dtype=torch.int64, device=dev)
    scr = ops._scratch(dev, L.srm2_plan_pack_scratch_bytes(nev, K), 'plan_pack')
    p = lambda t: t.data_ptr() if t.numel() else 0
    with torch.cuda.device(dev):
        st = L.srm2_plan_pack(p(ev_slot), p(rep), p(evf_slots), p(evl_ids), p(ev_dyn), nev, K, p(loc), loc.numel(), p(F_row), nF, int(nFa), p(S_row), nS,
                              p(c_slots), nc, p(L_ids), nL, p(a_ids), na, mat_top.data_ptr(), log_top.data_ptr(), live.data_ptr(),
                              p(evM_slot), p(evl_src), flat.data_ptr(), scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'plan_pack')
    return SimpleNamespace(evM_slot=evM_slot, evl_src=evl_src, flat=flat, parts=parts)


# ------------------------------------------------------------------------------------------------------------------
# The whole per-step plan on the fused kernels.
I32, I64, I8 = torch.int32, torch.int64, torch.int8
C_HIT, C_NADM, C_NAPP, C_NCMP, C_LADM, C_LAPP, C_LCMP, C_FADM, C_FNADM, C_S = range(10)      # srm2/elara.py:32


def plan(pl, s, u, u_nexts):
    """`ELARAPlanner.plan(s, u, u_nexts)` (reference: srm2/elara.py:209-414) on this library's kernels: classification and
    class partition, eviction candidates, directory call A, admissions, directory call B and the packing of the host work
    lists are seven calls into the library instead of ~230 small tensor operations.  `pl` is the reference's planner object
    (its state tensors and counters are read and updated exactly as its own plan() does; it must have been built with
    dir_impl='cpp' and its `dx` must be this library's dir_ext()).  Returns a Plan with the same fields and values.

    Host synchronisations: the one read of the eviction-candidate and class counts (srm2/elara.py:242) and the one
    device-to-host copy of the work lists (:406) remain, because the reference's Plan carries tensors whose SHAPES depend
    on those counts; the rare paths (preemption :248-253, overflow un-admission :254-259) add theirs only when they run,
    as in the reference.  To use it:  ELARAPlanner.plan = elara_b200.planner.plan."""
    d, K, MAT = pl.d, pl.Kmax, pl.MAT
    if not hasattr(pl.dx, 'admit'):
        raise RuntimeError("planner.plan needs this library's directory (pl.dx = elara_b200.ops.dir_ext())")
    n = u.numel()
    if pl.evl_mode == 2 and not pl.evict_logs and pl.gate is not None and pl.gate():         # :212-213
        pl.evict_logs = True
        pl.stats['evl_on_step'] = s
    ttl, want_T = pl.dyn == 'ttl', pl.st_mode == 'T'
    r = plan_classify(u, u_nexts, pl.slot_of, pl.last_seen, pl.code, pl.kthr, pl.toff, s, K, ttl, want_T)      # :214-219, 229-240
    e = evict_candidates(u_nexts, pl.slot_of, pl.pinned, pl.dyn_slots, pl.slot_row, pl.last_seen, s, ttl)    # :220-228, 245
    sl, in_next, admit, c, cls, order = r.sl, r.in_next, r.admit, r.c, r.cls, r.order
    vals = torch.cat([e.n_exp, r.counts]).tolist()                                            # the one host sync (:242)
    pl.stats['syncs'] += 1
    n_exp, counts = vals[0], vals[1:]
    n_adm = counts[C_NADM] + counts[C_LADM] + counts[C_FADM]
    ev_slot, keep_dyn = e.parted[:n_exp], e.parted[n_exp:]                                    # :246
    need = n_adm - (pl.n_free + n_exp)
    barrier = False
    if need > 0 and keep_dyn.numel():           # preempt residents that the pipeline window does not need (rare, :248-253)
        pre = ~e.protect[keep_dyn]
        n_pre = int(pre.sum()); pl.stats['syncs'] += 1
        take = min(need, n_pre)
        if take:
            o2 = torch.argsort((~pre).to(I8), stable=True)
            ev_slot = torch.cat([ev_slot, keep_dyn[o2[:take]]]); keep_dyn = keep_dyn[o2[take:]]
            n_exp += take; need -= take; pl.stats['preempt'] = pl.stats.get('preempt', 0) + take
    if need > 0:                                # overflow: un-admit, classify again with that admission mask (rare, :254-259)
        pri = (~admit).to(I32) * 4 + admit.to(I32) * (2 - 2 * in_next.to(I32))
        oo = torch.argsort(pri, stable=True); drop = oo[n_adm - need:n_adm]
        n_carry_drop = int(in_next[drop].sum()); pl.stats['syncs'] += 1
        admit[drop] = False; pl.stats['overflow'] += need; n_adm -= need; barrier = n_carry_drop > 0
        r = plan_classify(u, u_nexts, pl.slot_of, pl.last_seen, pl.code, pl.kthr, pl.toff, s, K, ttl, want_T, admit=admit)
        cls, order = r.cls, r.order
        counts = r.counts.tolist(); pl.stats['syncs'] += 1
    b_ = [0]
    for x in counts:
        b_.append(b_[-1] + x)
    rng = lambda lo, hi: order[b_[lo]:b_[hi + 1]]                                             # :260-263
    p = SimpleNamespace(); p.s = s; p.u = u; p.n = n; p.barrier = barrier
    hp = rng(C_HIT, C_HIT); p.hit_pos, p.hit_slot = hp, sl[hp].long()
    Npos, Lpos, Fpos, Spos = rng(C_NADM, C_NCMP), rng(C_LADM, C_LCMP), rng(C_FADM, C_FNADM), rng(C_S, C_S)
    p.N_pos, p.N_row = Npos, u[Npos]; p.L_pos, p.L_row = Lpos, u[Lpos]; p.L_cnt = c[Lpos].to(I32)
    p.F_pos, p.F_row = Fpos, u[Fpos]; p.S_pos, p.S_row = Spos, u[Spos]
    nNa, nNp, nNc, nLa, nLp, nLc, nFa, nFn = counts[1:9]
    assert nNa + nLa + nFa == n_adm, (nNa, nLa, nFa, n_adm)
    stv = [pl.code, pl.loc, pl.ent, pl.lstep, pl.lfree, pl.n_lfree, pl.log_top, pl.mat_top, pl.live,
           pl.adm_c0, pl.rj, pl.pstep, pl.kthr, pl.toff, pl.slot_of, pl.slot_row, pl.rok]                          # :275-277
    pv = [pl.R, K, pl.log_cap, pl.n0, pl.Cdyn, MAT, pl.mat_trash, int(pl.evict_logs)]
    (p.L_steps, L_ids, p.hrec_dyn, p.hrec_j, ev_row, rep, evl_ids, evf_slots, p.ev_dyn) = pl.dx.elara_dir_a(
        stv, pv, p.hit_slot, p.L_row, p.L_cnt, ev_slot, s)                                     # :278-279
    p.ev_slot, p.ev_row, p.ev_rep = ev_slot, ev_row, rep
    nev = ev_slot.numel()
    # ---- admissions (:345-367) ----
    pool_free = torch.cat([pl.free, ev_slot]); nf = pl.n_free + nev
    adm_slots = pool_free[nf - n_adm:]; pl.free = pool_free[:nf - n_adm]; pl.n_free = nf - n_adm
    adm_rows = torch.cat([p.N_row[:nNa], p.L_row[:nLa], p.F_row[:nFa]])
    ar = lambda a_, b2: torch.arange(a_, b2, device=d)
    ix = {'N_adm': ar(0, nNa), 'N_app': ar(nNa, nNa + nNp), 'N_cmp': ar(nNa + nNp, nNa + nNp + nNc),
          'L_adm': ar(0, nLa), 'L_app': ar(nLa, nLa + nLp), 'L_cmp': ar(nLa + nLp, nLa + nLp + nLc),
          'F_adm': ar(0, nFa), 'F_nadm': ar(nFa, nFa + nFn)}
    ix['N_upd'] = torch.cat([ix['N_adm'], ix['N_cmp']]); ix['L_upd'] = torch.cat([ix['L_adm'], ix['L_cmp']])
    ix['N_adm_slot'] = adm_slots[:nNa]; ix['L_adm_slot'] = adm_slots[nNa:nNa + nLa]; ix['F_adm_slot'] = adm_slots[nNa + nLa:]
    p.ix = ix; p.L_off = torch.cumsum(p.L_cnt.long(), 0) - p.L_cnt.long()
    lazy_n = nNa + nLa
    p.adm_rec_dyn = adm_slots[:lazy_n] - pl.n0 if pl.evict_logs else torch.full((lazy_n,), pl.Cdyn, dtype=I64, device=d)
    if n_adm:
        pl.dx.admit(stv, pv, adm_rows, adm_slots, lazy_n, s)                                  # :358-366 as one kernel
    pl.dyn_slots = torch.cat([keep_dyn, adm_slots])
    # ---- appends and compactions (:369-374) ----
    a_rows = torch.cat([p.N_row[nNa:nNa + nNp], p.L_row[nLa:nLa + nLp]])
    a_k = torch.cat([torch.zeros(nNp, dtype=I64, device=d), p.L_cnt[nLa:nLa + nLp].long()])
    c_rows = torch.cat([p.N_row[nNa + nNp:], p.L_row[nLa + nLp:]])
    c_cnt = torch.cat([torch.zeros(nNc, dtype=I64, device=d), p.L_cnt[nLa + nLp:].long()])
    a_ids, c_slots = pl.dx.elara_dir_b(stv, pv, a_rows, a_k, c_rows, c_cnt, s)
    pl.tcount[u] = torch.clamp(pl.tcount[u].to(torch.int16) + 1, max=255).to(torch.uint8)      # :387
    # ---- packed eviction outputs and host work lists, one device-to-host copy (:389-410) ----
    p.evl = bool(pl.evict_logs)
    k = pack(ev_slot, rep, evf_slots, evl_ids, p.ev_dyn, K, pl.loc, p.F_row, p.S_row, nFa, c_slots, L_ids, a_ids,
             pl.mat_top, pl.log_top, pl.live)
    p.evM_slot, p.evl_src = (k.evM_slot, k.evl_src) if nev else (p.ev_slot, torch.empty(0, dtype=I64, device=d))
    flat = k.flat.cpu(); pl.stats['syncs'] += 1
    p.cpu = {}; o = 0
    for name, m in k.parts:
        p.cpu[name] = flat[o:o + m]; o += m
    p.cpu['nev'] = nev
    p.cpu['nE'] = int((p.cpu['EVL_ids'] >= 0).sum())
    p.cpu['n_rep'] = int(p.cpu['tops'][3])
    st = pl.stats; st['adm'] += n_adm; st['ev'] += nev; st['hits'] += counts[C_HIT]
    st['N'] += Npos.numel(); st['L'] += Lpos.numel(); st['F'] += Fpos.numel(); st['S'] += Spos.numel()
    st['compactions'] += nNc + nLc; st['appends'] += nNp + nLp
    return p
