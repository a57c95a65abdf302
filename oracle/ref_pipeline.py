"""Driver of the reference's own planner + executor (srm2/elara.py:107-604) on the GPU, stock or with this library's
kernels substituted the way a maintainer would re-point them.

TEST INFRASTRUCTURE, like everything under oracle/: used by the parity tests and by the comparison figures of bench.py;
the shipped package never imports it.  Needs the reference's Python package staged in oracle/_ref/srm2 beside its compiled
extensions (oracle/build_ref.py).
"""
import collections
import sys
import time
from pathlib import Path

import numpy as np
import torch

REF = Path(__file__).resolve().parent / '_ref'
HYP = (1e-3, 0.9, 0.999, 1e-8)


def load_reference():
    """-> dict of the reference's modules with its two compiled extensions already loaded (no JIT build), or None."""
    if not (REF / 'srm2' / 'ops.py').exists():
        return None
    from . import oracle as O
    E, Dx = O.ref_cpu(), O.ref_dir()
    if E is None or Dx is None:
        return None
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import srm2.ops as rops
    rops._ext, rops._dir = E, Dx               # what ext() / dir_ext() return once loaded (srm2/ops.py:19-39)
    import srm2.gpu_ops as rgpu
    import srm2.elara as relara
    import srm2.executor as rexec
    import srm2.elara_kernels as rk
    return dict(ops=rops, gpu_ops=rgpu, elara=relara, executor=rexec, elara_kernels=rk, E=E, Dx=Dx)


def run_elara(ref, dev, substituted, R, C, dyn_slots, D, K, batch, steps, seed=42, L=8, depth=3, fused_executor=False, fused_plan=False):
    """One training-shaped run of the reference's planner + executor (single thread, default stream, the loop of
    srm2/train.py:409-444 without the dense model: the reduced gradient of a step is a seeded random matrix).
    substituted: gpu_adam / init_rows / replay_rows / ScalarTable / dir_ext re-pointed at this library;
    fused_executor: assemble() and update() through the fused kernels as well;
    fused_plan: ELARAPlanner.plan replaced by elara_b200.planner.plan (needs substituted=True: it uses this library's directory).
    -> (final state as a dict of tensors, planner statistics + 'ms_per_step' of the step loop)."""
    from elara_b200 import synth
    relara, rexec, rops = ref['elara'], ref['executor'], ref['ops']
    stock = dict(e_init=relara.init_rows, e_replay=relara.replay_rows, e_adam=relara.gpu_adam, x_init=rexec.init_rows,
                 x_replay=rexec.replay_rows, x_adam=rexec.gpu_adam, x_table=rexec.ScalarTable, dir_ext=rops.dir_ext)
    if substituted:        # the re-pointing a maintainer does (the names the reference's modules resolve at call time)
        import elara_b200.ops as b_ops
        import elara_b200.gpu_ops as b_gpu
        relara.init_rows = rexec.init_rows = b_gpu.init_rows
        relara.replay_rows = rexec.replay_rows = b_gpu.replay_rows
        relara.gpu_adam = rexec.gpu_adam = b_ops.gpu_adam
        rexec.ScalarTable = b_gpu.ScalarTable
        rops.dir_ext = b_ops.dir_ext
    stock_update, stock_assemble, stock_plan = relara.ELARAExecutor.update, relara.ELARAExecutor.assemble, relara.ELARAPlanner.plan
    if fused_plan:
        from elara_b200 import planner as b_planner
        relara.ELARAPlanner.plan = b_planner.plan
    if fused_executor:     # the executor's GPU glue as well: assemble and update through the fused kernels
        from elara_b200 import executor_ops
        import elara_b200.gpu_ops as b_gpu

        def assemble(self, p):        # srm2/elara.py:471-489 with its body (479-489) replaced by one call
            self._check()
            ev = self.staged[p.s][0]; ev.wait()
            self._check()
            (sw, ff, lg), e = self.staged.pop(p.s)[1]
            cur = torch.cuda.current_stream(self.d); cur.wait_event(e)
            for t in (sw, ff, lg): t.record_stream(cur)
            cfg = self.cfg
            W, fullN, fullL = b_gpu.assemble(p.n, self.D, self.pool, p.hit_pos, p.hit_slot, p.N_pos, p.N_row, p.L_pos, p.L_row, lg, p.L_off,
                                             p.L_steps, p.L_cnt, self.Kw, cfg['seed'], cfg['bound'], self.table, ff, p.F_pos, sw, p.S_pos)
            return W, (fullN, fullL, ff)

        def update(self, p, G, bufs):  # srm2/elara.py:491-542 with lines 497-532 replaced by one call
            cfg, dev = self.cfg, self.d
            og_gpu, of_gpu, oe_gpu = executor_ops.update(self.pool, self.glog, G, p, bufs, cfg['lr'], cfg['b1'], cfg['b2'], cfg['eps'])
            og = torch.empty(og_gpu.shape, pin_memory=True); of = torch.empty(of_gpu.shape, pin_memory=True)
            oe = torch.empty(oe_gpu.shape, pin_memory=True)
            cur = torch.cuda.current_stream(dev); ev_c = torch.cuda.Event(); ev_c.record(cur)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(ev_c)
                for h, g_ in ((og, og_gpu), (of, of_gpu), (oe, oe_gpu)):
                    h.copy_(g_, non_blocking=True); g_.record_stream(self.d2h)
                out_ev = torch.cuda.Event(); out_ev.record(self.d2h)
            self.counts['d2h_bytes'] += (og.numel() + of.numel() + oe.numel()) * 4
            self.enqueue_update_ids(p.s, out_ev, og, of, oe, p.cpu)
        relara.ELARAExecutor.update, relara.ELARAExecutor.assemble = update, assemble
    try:
        sizes, offs = synth.table_sizes(R, 26, seed=seed)
        ids = [torch.from_numpy(synth.zipf_lookups(sizes, offs, batch, 1.1, seed, s + 1)).to(dev) for s in range(steps)]
        U = [torch.unique(i) for i in ids]
        # static hot set: the most frequent rows of the first ten batches
        head = torch.cat(ids[:10])
        uu, cc = torch.unique(head, return_counts=True)
        n0 = min(C - dyn_slots, uu.numel())
        static_rows = uu[torch.argsort(cc, descending=True, stable=True)[:n0]].sort().values
        bound = float(np.sqrt(1.0 / sizes.max()))
        cfg = dict(lr=HYP[0], b1=HYP[1], b2=HYP[2], eps=HYP[3], seed=seed, bound=bound, max_step=steps)
        pl = relara.ELARAPlanner(R, C, K, 'static', 'ttl', 'T', static_rows, L, dev, torch.from_numpy(offs),
                                 torch.full((26,), K, dtype=torch.int8), evict_logs=1, dir_impl='cpp')
        ex = relara.ELARAExecutor(R, D, cfg, pl, dev, threads=8, depth=depth)
        ex.load_static()
        gen = torch.Generator(device=dev).manual_seed(seed)
        for j in range(min(steps, L + 1)):
            pl.observe(j + 1, U[j])
        nxt = [0]
        plan_s = [0.0]

        def get_plan():
            s = nxt[0]
            nxt[0] += 1
            if s + L + 1 < steps:
                pl.observe(s + L + 2, U[s + L + 1])
            t_p = time.perf_counter()
            p = pl.plan(s + 1, U[s], [U[s + k] for k in range(1, depth) if s + k < steps])      # ends with its device-to-host copy
            plan_s[0] += time.perf_counter() - t_p
            if p.barrier:
                ex.mark_barrier(p.s)
            return p
        ahead = collections.deque()
        for _ in range(min(steps, depth - 1)):
            ahead.append(get_plan())
            ex.enqueue_gather(ahead[-1])
        torch.cuda.synchronize(dev)
        t_loop = time.perf_counter()
        for s in range(steps):
            p = ahead.popleft()
            if s + depth - 1 < steps:
                ahead.append(get_plan())
                ex.enqueue_gather(ahead[-1])
            W, bufs = ex.assemble(p)
            gW = torch.randn(p.n, D, device=dev, generator=gen) * 1e-3
            ex.update(p, gW, bufs)
        ex.drain()
        torch.cuda.synchronize(dev)
        ms_per_step = (time.perf_counter() - t_loop) * 1e3 / steps
        Kk, Lcap, Cdyn = pl.Kmax, pl.log_cap, pl.Cdyn
        nf = int(pl.n_lfree)
        ent = pl.ent[:R * Kk]
        live_ids = ent[ent >= 0].long().cpu()
        out = dict(code=pl.code, loc=pl.loc[:R], ent=ent, lstep=pl.lstep[:Lcap], lfree=pl.lfree[:nf], n_lfree=pl.n_lfree,
                   log_top=pl.log_top, mat_top=pl.mat_top, live=pl.live, adm_c0=pl.adm_c0, rj=pl.rj, pstep=pl.pstep[:Cdyn],
                   kthr=pl.kthr, toff=pl.toff, slot_of=pl.slot_of, slot_row=pl.slot_row, rok=pl.rok,
                   free=pl.free, dyn_slots=pl.dyn_slots, tcount=pl.tcount, pool=ex.pool, glog=ex.glog[:Cdyn],
                   mat=ex.store.mat[:int(pl.mat_top)].clone(), live_logs=ex.store.logs[live_ids].clone(),
                   W_last=W)
        stats = dict(pl.stats)
        stats['ms_per_step'] = ms_per_step
        stats['plan_ms_per_step'] = plan_s[0] * 1e3 / steps
        ex.close()
        return out, stats
    finally:
        relara.init_rows, relara.replay_rows, relara.gpu_adam = stock['e_init'], stock['e_replay'], stock['e_adam']
        rexec.init_rows, rexec.replay_rows, rexec.gpu_adam = stock['x_init'], stock['x_replay'], stock['x_adam']
        rexec.ScalarTable, rops.dir_ext = stock['x_table'], stock['dir_ext']
        relara.ELARAExecutor.update, relara.ELARAExecutor.assemble = stock_update, stock_assemble
        relara.ELARAPlanner.plan = stock_plan
