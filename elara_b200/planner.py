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
