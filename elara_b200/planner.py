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
