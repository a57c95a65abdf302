"""Golden vectors for the classification / partition part of the reference's ELARAPlanner.plan (srm2/elara.py:209-271):
the planner itself runs on CPU tensors (C++ directory compiled by oracle/build_ref.py); before every plan() call the
state it reads (slot_of, last_seen, code, pinned, dyn_slots, slot_row) and its inputs (u, the look-ahead lists) are recorded, after it the position
lists and eviction candidates of the returned Plan and the planner's new list of dynamic slots.  Seeded synthetic ids; nothing here is taken from a dataset.

    python tests/golden/make_plan_golden.py [--ref <checkout of the reference>]
"""
import argparse
import os
import sys
from pathlib import Path

os.environ['TRITON_INTERPRET'] = '1'
HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(HERE))

import numpy as np   # noqa: E402
import torch         # noqa: E402


def gen_plan(elara, out, name, dyn, st_mode, kthr, steps=20, seed=5):
    from make_golden import zipf_ids
    R, C, K, L, depth = 3000, 320, 3, 4, 3
    sizes = [40, 260, 900, 1800]
    toff = np.concatenate([[0], np.cumsum(sizes)[:-1]]).astype(np.int64)
    rng = np.random.default_rng(seed)
    U = [torch.from_numpy(np.unique(zipf_ids(rng, toff, sizes, 96, 1.1))) for _ in range(steps)]
    cnt = np.zeros(R, np.int64)
    for u in U[:4]:
        cnt[u.numpy()] += 1
    static_rows = torch.from_numpy(np.sort(np.argsort(-cnt, kind='stable')[:200]).astype(np.int64))
    pl = elara.ELARAPlanner(R, C, K, 'static', dyn, st_mode, static_rows, L, 'cpu', torch.from_numpy(toff),
                            torch.tensor(kthr, dtype=torch.int8), evict_logs=1, dir_impl='cpp')
    pl.code[static_rows] = pl.MAT
    rec = {}
    real = pl.dx

    class Recorder:                                   # the directory calls inside plan(): their outputs feed the packing
        def elara_dir_a(self, *a):
            rec['a'] = real.elara_dir_a(*a); return rec['a']

        def elara_dir_b(self, *a):
            rec['b'] = real.elara_dir_b(*a); return rec['b']
    pl.dx = Recorder()
    save = {'K': np.array(K), 'ttl': np.array(int(dyn == 'ttl')), 'want_T': np.array(int(st_mode == 'T')), 'steps': np.array(steps),
            'toff': toff, 'kthr': np.array(kthr, np.int8)}
    for j in range(min(steps, L + 1)):
        pl.observe(j + 1, U[j])
    for s0 in range(steps):
        if s0 + L + 1 < steps:
            pl.observe(s0 + L + 2, U[s0 + L + 1])
        s = s0 + 1
        nexts = [U[s0 + k] for k in range(1, depth) if s0 + k < steps]
        save[f's{s}_u'] = U[s0].numpy()
        save[f's{s}_n_next'] = np.array(len(nexts))
        for q, un in enumerate(nexts):
            save[f's{s}_next{q}'] = un.numpy()
        for k in ('slot_of', 'last_seen', 'code', 'pinned', 'dyn_slots', 'slot_row'):
            save[f's{s}_{k}'] = getattr(pl, k).numpy().copy()
        overflow0 = pl.stats.get('overflow', 0)
        p = pl.plan(s, U[s0], nexts)
        save[f's{s}_overflow'] = np.array(int(pl.stats.get('overflow', 0) != overflow0))   # un-admission ran: not the plain classification
        for k in ('hit_pos', 'hit_slot', 'N_pos', 'L_pos', 'F_pos', 'S_pos', 'L_cnt'):
            save[f's{s}_{k}'] = getattr(p, k).numpy()
        save[f's{s}_ev_slot'] = p.ev_slot.numpy()                      # eviction candidates, and what stayed (head of the new list)
        save[f's{s}_dyn_slots_after'] = pl.dyn_slots.numpy().copy()
        save[f's{s}_preempt'] = np.array(int(pl.stats.get('preempt', 0)))
        # packing of the eviction outputs and host work lists (srm2/elara.py:389-407): inputs ...
        for nm, t in zip(('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn'), rec['a']):
            if nm in ('L_ids', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn'):
                save[f's{s}_pk_{nm}'] = t.numpy().copy()
        save[f's{s}_pk_a_ids'] = rec['b'][0].numpy().copy(); save[f's{s}_pk_c_slots'] = rec['b'][1].numpy().copy()
        save[f's{s}_pk_loc'] = pl.loc.numpy().copy()
        save[f's{s}_pk_tops'] = np.array([int(pl.mat_top), int(pl.log_top), int(pl.live)], np.int64)
        save[f's{s}_pk_F_row'] = p.F_row.numpy(); save[f's{s}_pk_S_row'] = p.S_row.numpy()
        save[f's{s}_pk_nFa'] = np.array(p.ix['F_adm'].numel())
        # ... and outputs
        save[f's{s}_pk_evM_slot'] = p.evM_slot.numpy(); save[f's{s}_pk_evl_src'] = p.evl_src.numpy()
        for k_ in ('S_slot', 'F_slot', 'L_ids', 'A_ids', 'W_slot', 'EVL_ids', 'tops'):
            save[f's{s}_pk_cpu_{k_}'] = p.cpu[k_].numpy().copy()
        for X in ('N', 'L'):
            save[f's{s}_{X}_n_adm'] = np.array(p.ix[X + '_adm'].numel())
    print(name, {k: v for k, v in pl.stats.items() if v})
    np.savez_compressed(out / f'{name}.npz', **save)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref', default=os.environ.get('SRM2_REFERENCE'), required=not os.environ.get('SRM2_REFERENCE'), help='the reference checkout (or set SRM2_REFERENCE)')
    a = ap.parse_args()
    sys.path.insert(0, a.ref)
    from oracle import oracle as O
    assert O.ref_cpu() is not None and O.ref_dir() is not None, 'run python oracle/build_ref.py first'
    import srm2.ops as ops
    ops._ext = O.ref_cpu(); ops._dir = O.ref_dir()
    import srm2.elara as elara
    gen_plan(elara, HERE, 'plan_ttl_T', 'ttl', 'T', [3, 3, 2, 1])
    gen_plan(elara, HERE, 'plan_carry_S', 'carry', 'S', [3, 2, 3, 0], seed=9)


if __name__ == '__main__':
    main()
