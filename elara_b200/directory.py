"""Mirror of the reference's directory extension `srm2.ops.dir_ext()` (reference: srm2/ops.py:32-39 loading
srm2/csrc/elara_dir.cpp) on the fused sm_100a kernels of libsrm2_b200.so, plus the pool-slot admissions that the
reference performs in torch between the two calls (srm2/elara.py:358-366)."""
import ctypes as C

import torch

from . import _lib

_FIELDS = ('code', 'loc', 'ent', 'lstep', 'lfree', 'n_lfree', 'log_top', 'mat_top', 'live', 'adm_c0', 'rj', 'pstep', 'kthr', 'toff',
           'slot_of', 'slot_row', 'rok')
_DTYPES = (torch.int8, torch.int32, torch.int32, torch.int32, torch.int32, torch.int64, torch.int64, torch.int64, torch.int64, torch.int8,
           torch.int8, torch.int32, torch.int8, torch.int64, torch.int32, torch.int64, torch.int8)


class _State(C.Structure):
    _fields_ = [(k, C.c_void_p) for k in _FIELDS] + [(k, C.c_int64) for k in ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl', 'T')]


def _state(st, pv):
    """st: the reference's list of 17 tensors; pv: [R, K, Lcap, n0, Cdyn, MAT, trash, evict_logs] (srm2/elara.py:275-277)."""
    if len(st) != 17 or len(pv) != 8:
        raise RuntimeError('directory state must be 17 tensors and 8 integers')
    s = _State()
    for name, dt, t in zip(_FIELDS, _DTYPES, st):
        if not t.is_cuda:
            raise RuntimeError(f'{name} must be a CUDA tensor: this library has no CPU path')
        if t.dtype != dt or not t.is_contiguous():
            raise TypeError(f'{name} must be a contiguous {dt} tensor')
        setattr(s, name, t.data_ptr())
    for name, v in zip(('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl'), pv):
        setattr(s, name, int(v))
    s.T = st[13].numel()
    return s


def _i64(t, name):
    if t.dtype != torch.int64:
        raise TypeError(f'{name} must be int64')
    return t.contiguous()


class _DirExt:
    """Same call signatures, argument meaning and return values as the reference's pybind module."""

    def __init__(self):
        self._scr = {}

    def _scratch(self, dev, items):
        L = _lib.lib()
        nb = L.srm2_dir_scratch_bytes(int(items))
        buf = self._scr.get(dev)
        if buf is None or buf.numel() < nb:
            new = torch.zeros(max(nb, 4096) * 2, dtype=torch.uint8, device=dev)
            if buf is not None:      # the head of the buffer holds the sticky status word of the plan step under way
                new[:4096].copy_(buf[:4096])
            self._scr[dev] = buf = new
        return buf

    def elara_dir_a(self, st, pv, hs, L_row, L_cnt, ev_slot, s):
        d = _state(st, pv)
        dev = st[0].device
        K = int(pv[1])
        hs, L_row, ev_slot = _i64(hs, 'hs'), _i64(L_row, 'L_row'), _i64(ev_slot, 'ev_slot')
        if L_cnt.dtype != torch.int32:
            raise TypeError('L_cnt must be int32')
        L_cnt = L_cnt.contiguous()
        nh, nL, nev = hs.numel(), L_row.numel(), ev_slot.numel()
        o = dict(L_steps=torch.empty(nL, K, dtype=torch.int32, device=dev), L_ids=torch.empty(nL, K, dtype=torch.int32, device=dev),
                 hrec_dyn=torch.empty(nh, dtype=torch.int64, device=dev), hrec_j=torch.empty(nh, dtype=torch.int64, device=dev),
                 ev_row=torch.empty(nev, dtype=torch.int64, device=dev), rep=torch.empty(nev, dtype=torch.bool, device=dev),
                 evl_ids=torch.empty(nev, K, dtype=torch.int64, device=dev), evf_slots=torch.empty(nev, dtype=torch.int64, device=dev),
                 ev_dyn=torch.empty(nev, dtype=torch.int64, device=dev))
        scr = self._scratch(dev, nev)
        with torch.cuda.device(dev):
            rc = _lib.lib().srm2_dir_a(C.byref(d), _lib.ptr(hs), nh, _lib.ptr(L_row), _lib.ptr(L_cnt), nL, _lib.ptr(ev_slot), nev, int(s),
                                       *[_lib.ptr(o[k]) for k in ('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids',
                                                                  'evf_slots', 'ev_dyn')],
                                       scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
        _lib.check(rc, 'elara_dir_a')
        return [o[k] for k in ('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn')]

    def admit(self, st, pv, adm_rows, adm_slots, lazy_n, s):
        """The torch statements of srm2/elara.py:358-366 as one kernel (slot_of, slot_row, adm_c0, rj, rok, pstep)."""
        d = _state(st, pv)
        dev = st[0].device
        adm_rows, adm_slots = _i64(adm_rows, 'adm_rows'), _i64(adm_slots, 'adm_slots')
        if adm_rows.numel() != adm_slots.numel():
            raise RuntimeError('adm_rows and adm_slots differ in length')
        scr = self._scratch(dev, 0)
        with torch.cuda.device(dev):
            rc = _lib.lib().srm2_dir_admit(C.byref(d), _lib.ptr(adm_rows), _lib.ptr(adm_slots), adm_rows.numel(), int(lazy_n), int(s),
                                           scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
        _lib.check(rc, 'dir_admit')

    def elara_dir_b(self, st, pv, a_rows, a_k, c_rows, c_cnt, s):
        d = _state(st, pv)
        dev = st[0].device
        a_rows, a_k, c_rows, c_cnt = _i64(a_rows, 'a_rows'), _i64(a_k, 'a_k'), _i64(c_rows, 'c_rows'), _i64(c_cnt, 'c_cnt')
        na, nc = a_rows.numel(), c_rows.numel()
        if a_k.numel() != na or c_cnt.numel() != nc:
            raise RuntimeError('a_k / c_cnt length mismatch')
        a_ids = torch.empty(na, dtype=torch.int64, device=dev)
        c_slots = torch.empty(nc, dtype=torch.int64, device=dev)
        scr = self._scratch(dev, max(na, nc))
        with torch.cuda.device(dev):
            rc = _lib.lib().srm2_dir_b(C.byref(d), _lib.ptr(a_rows), _lib.ptr(a_k), na, _lib.ptr(c_rows), _lib.ptr(c_cnt), nc, int(s),
                                       _lib.ptr(a_ids), _lib.ptr(c_slots), scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
        _lib.check(rc, 'elara_dir_b')
        return [a_ids, c_slots]

    def status(self, device):
        """Sticky error word of the current plan step (0 = no index was out of range); synchronises."""
        scr = self._scr.get(device)
        if scr is None:
            return 0
        out = torch.zeros(1, dtype=torch.int32, device=device)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().srm2_dir_status(scr.data_ptr(), out.data_ptr(), _lib.stream_of(device)), 'dir_status')
        return int(out.item())


_dir = None


def dir_ext():
    global _dir
    if _dir is None:
        _lib.lib()
        _dir = _DirExt()
    return _dir
