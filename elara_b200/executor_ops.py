"""The GPU half of the reference executor's update step in three kernel launches
(reference: ELARAExecutor.update, srm2/elara.py:491-531).

`update(pool, glog, G, p, bufs, lr, b1, b2, eps)` takes the reference's own objects — the pool [C,3,D], the resident
history tensor glog [Cdyn+1, K, D], the reduced gradients G [n, D], the planner's Plan `p` and the buffers that
assemble() returned — applies every pool and history update of the step and returns the three tensors the reference
copies to the host next (og, of, oe), with the same contents in the same order.  In the reference the body of
ELARAExecutor.update up to the pinned copies (srm2/elara.py:497-532) becomes

    og_gpu, of_gpu, oe_gpu = executor_ops.update(self.pool, self.glog, G, p, bufs, cfg['lr'], cfg['b1'], cfg['b2'], cfg['eps'])
"""
import torch

from . import _lib, ops


def update(pool, glog, G, p, bufs, lr, b1, b2, eps):
    if not pool.is_cuda:
        raise RuntimeError('pool must be a CUDA tensor: this library has no CPU path')
    fullN, fullL, ff = bufs
    dev, D = pool.device, pool.shape[2]
    ix = p.ix
    nNa, nNp, nNc = ix['N_adm'].numel(), ix['N_app'].numel(), ix['N_cmp'].numel()
    nLa, nLp, nLc = ix['L_adm'].numel(), ix['L_app'].numel(), ix['L_cmp'].numel()
    nFa, nFn = ix['F_adm'].numel(), ix['F_nadm'].numel()
    nS, n_hit = p.S_pos.numel(), p.hit_pos.numel()
    n_evM = p.ev_slot.numel() - int(p.cpu['n_rep'])         # rows going to M come first in evM_slot (srm2/elara.py:505)
    n_evl = int(p.cpu['nE'])
    og = torch.empty(nS + nNp + nLp, D, device=dev)
    of = torch.empty(nNc + nLc + nFn + n_evM, 3, D, device=dev)
    oe = torch.empty(n_evl, D, device=dev)
    tensors = dict(G=G, pool=pool, glog=glog, fullN=fullN, fullL=fullL, ff=ff)
    for name, t in tensors.items():
        if t is not None and t.numel() and (t.dtype != torch.float32 or not t.is_contiguous() or t.device != dev):
            raise RuntimeError(f'{name} must be a contiguous float32 tensor on the device of pool')
    idx = dict(hit_pos=p.hit_pos, hit_slot=p.hit_slot, hrec_dyn=getattr(p, 'hrec_dyn', None), hrec_j=getattr(p, 'hrec_j', None),
               S_pos=p.S_pos, N_pos=p.N_pos, L_pos=p.L_pos, F_pos=p.F_pos, evM_slot=p.evM_slot, evl_src=p.evl_src,
               N_adm_slot=ix['N_adm_slot'], L_adm_slot=ix['L_adm_slot'], F_adm_slot=ix['F_adm_slot'], adm_rec_dyn=p.adm_rec_dyn)
    keep = []
    for name, t in idx.items():
        if t is not None and t.numel():
            if t.dtype != torch.int64 or t.device != dev:
                raise RuntimeError(f'{name} must be an int64 tensor on the device of pool')
            if not t.is_contiguous():
                t = t.contiguous()
                keep.append(t)
            idx[name] = t
    if len(p.evM_slot) < n_evM or len(p.evl_src) < n_evl:
        raise RuntimeError('the plan lists fewer evicted slots / history entries than its counts say')
    ptr = lambda t: t.data_ptr() if t is not None and t.numel() else 0
    U = _lib.Update()
    U.D, U.K, U.evl = D, (glog.shape[1] if glog is not None and glog.dim() == 3 else 0), int(bool(p.evl))
    U.G, U.pool, U.glog = ptr(G), ptr(pool), ptr(glog)
    sc = ops._scalars(lr, b1, b2, eps, p.s)
    for k in range(8):
        U.sc[k] = sc[k]
    U.hit_pos, U.hit_slot, U.hrec_dyn, U.hrec_j, U.n_hit = ptr(idx['hit_pos']), ptr(idx['hit_slot']), ptr(idx['hrec_dyn']), ptr(idx['hrec_j']), n_hit
    U.S_pos, U.n_S = ptr(idx['S_pos']), nS
    U.fullN, U.N_pos, U.nNa, U.nNp, U.nNc = ptr(fullN), ptr(idx['N_pos']), nNa, nNp, nNc
    U.fullL, U.L_pos, U.nLa, U.nLp, U.nLc = ptr(fullL), ptr(idx['L_pos']), nLa, nLp, nLc
    U.ff, U.F_pos, U.nFa, U.nFn = ptr(ff), ptr(idx['F_pos']), nFa, nFn
    U.evM_slot, U.n_evM, U.evl_src, U.n_evl = ptr(idx['evM_slot']), n_evM, ptr(idx['evl_src']), n_evl
    U.N_adm_slot, U.L_adm_slot, U.F_adm_slot, U.adm_rec_dyn = ptr(idx['N_adm_slot']), ptr(idx['L_adm_slot']), ptr(idx['F_adm_slot']), ptr(idx['adm_rec_dyn'])
    U.og, U.of, U.oe = ptr(og), ptr(of), ptr(oe)
    import ctypes as C
    with torch.cuda.device(dev):
        st = _lib.lib().srm2_executor_update_f32(C.byref(U), _lib.stream_of(dev))
    _lib.check(st, 'executor_update')
    return og, of, oe
