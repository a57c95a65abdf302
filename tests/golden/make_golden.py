"""Generate the golden vectors under tests/golden/ from the reference implementation itself.

Run in a container that has the reference checkout (read-only) and the compiled reference sources
(`python oracle/build_ref.py`):

    python tests/golden/make_golden.py [--ref <checkout of the reference>]

What produces each file:
  adam_*.npz       the reference's C++ cpu_adam / adam_scalars (srm2/csrc/srm2_cpu.cpp) AND its Triton
                   gpu_adam (srm2/ops.py) run by the Triton CPU interpreter; the two must agree.
  init_*.npz       the reference's Triton init_rows (srm2/gpu_ops.py) under the Triton CPU interpreter.
  replay_*.npz     the reference's Triton replay_rows under the interpreter, plus its eager path
                   (init_rows then cpu_adam at each logged step, as tests/test_replay.py does).
  dir_*.npz        the reference's ELARAPlanner (srm2/elara.py) on CPU tensors with the C++ directory
                   (srm2/csrc/elara_dir.cpp): inputs, outputs and state of every directory call.

The inputs are seeded synthetic data; nothing here is taken from a dataset.
"""
import argparse
import os
import sys
import zlib
from pathlib import Path

os.environ['TRITON_INTERPRET'] = '1'          # must precede the first triton import
HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np   # noqa: E402
import torch         # noqa: E402


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def gen_adam(O, ops, out):
    E = O.ref_cpu()
    for name, (R, D, n, steps) in {'adam_d16': (512, 16, 160, 5), 'adam_d24': (300, 24, 90, 4), 'adam_d128': (256, 128, 64, 4)}.items():
        g = torch.Generator().manual_seed(1000 + D)
        state0 = torch.randn(R, 3, D, generator=g) * 0.05
        state0[:, 1:] = 0
        host = state0.clone(); trit = state0.clone()
        rows_l, grad_l, sc_l = [], [], []
        for step in range(1, steps + 1):
            rows = torch.randperm(R, generator=g)[:n].sort().values
            if step == 2:
                rows = rows[torch.randperm(n, generator=g)]        # unsorted order
            grad = torch.randn(n, D, generator=g) * (10.0 ** (step % 3 - 2))
            if step == 3:
                grad[0] = 0.0; grad[1, :4] = 1e-30; grad[2] = -0.0   # zero, tiny (subnormal v) and negative-zero gradients
            t = step * 7 if step > 2 else step
            E.cpu_adam(host, rows, grad, 1e-3, 0.9, 0.999, 1e-8, t, 4)
            ops.gpu_adam(trit, rows.to(torch.int32) if step % 2 else rows, grad, 1e-3, 0.9, 0.999, 1e-8, t)
            rows_l.append(rows.numpy()); grad_l.append(grad.numpy()); sc_l.append(np.array(E.adam_scalars(1e-3, 0.9, 0.999, 1e-8, t), np.float32))
        assert torch.equal(host, trit), 'reference CPU and Triton Adam disagree'
        np.savez_compressed(out / f'{name}.npz', state0=state0.numpy(), rows=np.stack(rows_l), grad=np.stack(grad_l),
                            scalars=np.stack(sc_l), steps=np.array([1, 2, 21, 28, 35][:steps]), state_out=host.numpy(),
                            hyper=np.array([1e-3, 0.9, 0.999, 1e-8]))
    # scalars for many steps and two hyper-parameter sets
    sets = [(1e-3, 0.9, 0.999, 1e-8), (0.05, 0.8, 0.99, 1e-6)]
    steps = np.array([1, 2, 3, 10, 50, 100, 1000, 12345, 10**6], np.int64)
    sc = np.array([[E.adam_scalars(*h, int(s)) for s in steps] for h in sets], np.float32)
    np.savez_compressed(out / 'adam_scalars.npz', hyper=np.array(sets), steps=steps, scalars=sc)


def gen_init_replay(O, ops, gpu_ops, out):
    E = O.ref_cpu()
    rows = torch.tensor([0, 1, 2, 5, 999_999, 3_999_999, 29_999_999, 2**31 - 1, 2**31, 2**32 - 1, 2**32, 2**32 + 7, 2**40 + 3],
                        dtype=torch.int64)
    res = {}
    for D in (16, 24, 64, 128):
        for seed, bound in ((1234, 0.01), (42, 0.01), (2**31 + 5, 0.0003162), (2**33 + 9, 0.5), (-3, 0.01)):
            res[f'D{D}_seed{seed}'] = gpu_ops.init_rows(rows, D, seed, bound).numpy()
            res[f'D{D}_seed{seed}_bound'] = np.array(bound)
    np.savez_compressed(out / 'init_rows.npz', rows=rows.numpy(), **res)

    for name, (D, K, n, smax) in {'replay_d64_k3': (64, 3, 96, 50), 'replay_d128_k3': (128, 3, 48, 1200), 'replay_d24_k2': (24, 2, 40, 9),
                                  'replay_d16_k4': (16, 4, 40, 30)}.items():
        g = torch.Generator().manual_seed(D * 100 + K)
        seed, bound = 1234, 0.01
        rws = torch.randint(0, 30_000_000, (n,), generator=g, dtype=torch.int64).unique(); n = rws.numel()
        rws[0] = 2**32 + 11
        cnt = torch.randint(0, K + 1, (n,), generator=g, dtype=torch.int32)
        steps = torch.zeros(n, K, dtype=torch.int32)
        for i in range(n):
            c = int(cnt[i])
            st = torch.randperm(smax, generator=g)[:c].sort().values + 1
            steps[i, :c] = st.to(torch.int32)
        offs = torch.cumsum(cnt.long(), 0) - cnt.long()
        logs = torch.randn(int(cnt.sum()), D, generator=g) * 1e-2
        table = gpu_ops.ScalarTable(1e-3, 0.9, 0.999, 1e-8, smax, 'cpu')
        rp = gpu_ops.replay_rows(rws, logs, offs, steps, cnt, D, K, seed, bound, table)
        # eager path of tests/test_replay.py:20-27 on the CPU kernel
        ec = gpu_ops.init_rows(rws, D, seed, bound).clone()
        for k in range(K):
            sel = (cnt > k).nonzero().flatten()
            for s_val in steps[sel, k].unique().tolist():
                idx = sel[steps[sel, k] == s_val]
                E.cpu_adam(ec, idx, logs[offs[idx] + k].contiguous(), 1e-3, 0.9, 0.999, 1e-8, s_val, 1)
        assert torch.equal(rp, ec), 'reference replay and eager Adam disagree'
        np.savez_compressed(out / f'{name}.npz', rows=rws.numpy(), logs=logs.numpy(), offs=offs.numpy(), steps=steps.numpy(),
                            cnt=cnt.numpy(), table=table.t.numpy(), out=rp.numpy(), meta=np.array([D, K, seed, smax]),
                            bound=np.array(bound), hyper=np.array([1e-3, 0.9, 0.999, 1e-8]))


# ---------------------------------------------------------------------------------------------
DIR_FIELDS = ('code', 'loc', 'ent', 'lstep', 'lfree', 'n_lfree', 'log_top', 'mat_top', 'live', 'adm_c0', 'rj', 'pstep',
              'kthr', 'toff', 'slot_of', 'slot_row', 'rok')


def zipf_ids(rng, toff, sizes, batch, alpha):
    """One lookup per table and sample, rank ~ truncated Zipf(alpha); sample-major flat ids."""
    cols = []
    for off, v in zip(toff, sizes):
        p = np.arange(1, v + 1, dtype=np.float64) ** -alpha
        p /= p.sum()
        cols.append(off + rng.choice(v, size=batch, p=p))
    return np.stack(cols, 1).reshape(-1).astype(np.int64)


def gen_dir(O, elara, out, name, evl, dyn, kthr, steps=36, seed=7):
    R, C, K, L, depth = 3000, 320, 3, 4, 3
    sizes = [40, 260, 900, 1800]
    toff = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
    rng = np.random.default_rng(seed)
    U = [torch.from_numpy(np.unique(zipf_ids(rng, toff, sizes, 96, 1.1))) for _ in range(steps)]
    cnt = np.zeros(R, np.int64)
    for u in U[:4]:
        cnt[u.numpy()] += 1
    n0 = 200
    static_rows = torch.from_numpy(np.sort(np.argsort(-cnt, kind='stable')[:n0]).astype(np.int64))
    pl = elara.ELARAPlanner(R, C, K, 'static', dyn, 'T', static_rows, L, 'cpu', torch.from_numpy(toff),
                            torch.tensor(kthr, dtype=torch.int8), evict_logs=evl, dir_impl='cpp')
    pl.code[static_rows] = pl.MAT            # what ELARAExecutor.load_static does (srm2/elara.py:439)

    def state():
        t = dict(code=pl.code, loc=pl.loc, ent=pl.ent, lstep=pl.lstep, lfree=pl.lfree, n_lfree=pl.n_lfree, log_top=pl.log_top,
                 mat_top=pl.mat_top, live=pl.live, adm_c0=pl.adm_c0, rj=pl.rj, pstep=pl.pstep, kthr=pl.kthr, toff=pl.toff,
                 slot_of=pl.slot_of, slot_row=pl.slot_row, rok=pl.rok)
        return {k: v.numpy().copy() for k, v in t.items()}

    pv = dict(R=R, K=K, Lcap=pl.log_cap, n0=pl.n0, Cdyn=pl.Cdyn, MAT=pl.MAT, trash=pl.mat_trash, evl=int(pl.evict_logs))

    def crcs(st):
        cmp = O.dir_comparable(st, pv)
        return np.array([zlib.crc32(np.ascontiguousarray(cmp[k]).tobytes()) for k in DIR_FIELDS], np.int64)

    rec = {}
    real = pl.dx

    class Recorder:
        def elara_dir_a(self, stv, pvv, hs, L_row, L_cnt, ev_slot, s):
            o = real.elara_dir_a(stv, pvv, hs, L_row, L_cnt, ev_slot, s)
            rec[f's{s}_a_in'] = (hs, L_row, L_cnt, ev_slot)
            rec[f's{s}_a_out'] = o
            rec[f's{s}_a_crc'] = crcs(state())
            return o

        def elara_dir_b(self, stv, pvv, a_rows, a_k, c_rows, c_cnt, s):
            rec[f's{s}_adm_crc'] = crcs(state())
            o = real.elara_dir_b(stv, pvv, a_rows, a_k, c_rows, c_cnt, s)
            rec[f's{s}_b_in'] = (a_rows, a_k, c_rows, c_cnt)
            rec[f's{s}_b_out'] = o
            rec[f's{s}_b_crc'] = crcs(state())
            return o

    pl.dx = Recorder()
    save = {'pv': np.array([pv[k] for k in ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl')], np.int64),
            'C': np.array(C), 'steps': np.array(steps)}
    for k, v in state().items():
        save[f'init_{k}'] = v
    for j in range(min(steps, L + 1)):
        pl.observe(j + 1, U[j])
    for s0 in range(steps):
        if s0 + L + 1 < steps:
            pl.observe(s0 + L + 2, U[s0 + L + 1])
        s = s0 + 1
        p = pl.plan(s, U[s0], [U[s0 + k] for k in range(1, depth) if s0 + k < steps])
        ix = p.ix
        nNa, nLa, nFa = ix['N_adm'].numel(), ix['L_adm'].numel(), ix['F_adm'].numel()
        adm_rows = torch.cat([p.N_row[:nNa], p.L_row[:nLa], p.F_row[:nFa]])
        adm_slots = torch.cat([ix['N_adm_slot'], ix['L_adm_slot'], ix['F_adm_slot']])
        hs, L_row, L_cnt, ev_slot = rec[f's{s}_a_in']
        save.update({f's{s}_hs': hs.numpy(), f's{s}_L_row': L_row.numpy(), f's{s}_L_cnt': L_cnt.numpy(), f's{s}_ev_slot': ev_slot.numpy()})
        for nm, t in zip(('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn'), rec[f's{s}_a_out']):
            save[f's{s}_o_{nm}'] = t.numpy()
        save[f's{s}_adm_rows'] = adm_rows.numpy(); save[f's{s}_adm_slots'] = adm_slots.numpy(); save[f's{s}_lazy_n'] = np.array(nNa + nLa)
        a_rows, a_k, c_rows, c_cnt = rec[f's{s}_b_in']
        save.update({f's{s}_a_rows': a_rows.numpy(), f's{s}_a_k': a_k.numpy(), f's{s}_c_rows': c_rows.numpy(), f's{s}_c_cnt': c_cnt.numpy()})
        save[f's{s}_o_a_ids'] = rec[f's{s}_b_out'][0].numpy(); save[f's{s}_o_c_slots'] = rec[f's{s}_b_out'][1].numpy()
        save[f's{s}_crc'] = np.stack([rec[f's{s}_a_crc'], rec[f's{s}_adm_crc'], rec[f's{s}_b_crc']])
        if s % 12 == 0 or s == steps:
            for k, v in state().items():
                if k not in ('kthr', 'toff'):
                    save[f's{s}_state_{k}'] = v
    print(name, 'stats', {k: v for k, v in pl.stats.items() if v}, 'live', int(pl.live), 'mat_top', int(pl.mat_top),
          'n_lfree', int(pl.n_lfree), 'log_top', int(pl.log_top))
    np.savez_compressed(out / f'{name}.npz', **save)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref', default=os.environ.get('SRM2_REFERENCE'), required=not os.environ.get('SRM2_REFERENCE'), help='the reference checkout (or set SRM2_REFERENCE)')
    a = ap.parse_args()
    sys.path.insert(0, a.ref)
    from oracle import oracle as O
    assert O.ref_cpu() is not None and O.ref_dir() is not None, 'run python oracle/build_ref.py first'
    import srm2.ops as ops
    ops._ext = O.ref_cpu(); ops._dir = O.ref_dir()      # the compiled reference sources, no JIT build dir needed
    import srm2.gpu_ops as gpu_ops
    import srm2.elara as elara
    gen_adam(O, ops, HERE)
    gen_init_replay(O, ops, gpu_ops, HERE)
    gen_dir(O, elara, HERE, 'dir_ttl_evl1', 1, 'ttl', [3, 3, 2, 1])
    gen_dir(O, elara, HERE, 'dir_ttl_evl0', 0, 'ttl', [3, 3, 3, 3], steps=24, seed=11)
    gen_dir(O, elara, HERE, 'dir_carry_evl1', 1, 'carry', [3, 2, 3, 0], steps=24, seed=13)


if __name__ == '__main__':
    main()
