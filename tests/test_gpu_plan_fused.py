"""The whole plan step on the fused kernels (elara_b200.planner.plan) against the reference's own ELARAPlanner.plan
(srm2/elara.py:209-414) on the GPU: two planner objects of the reference's class, the same seeded id stream; one runs the
stock plan() with the reference's compiled directory extension, the other has plan() replaced by this library's and `dx` by
this library's directory.  After every step every field of the two Plans is compared (tensors, index ranges, the host work
lists); at the end the planners' states.  The small pools make the rare paths run: preemption of residents
(srm2/elara.py:248-253) and overflow un-admission with the second classification (:254-259).
Skips when the reference's package is not staged in oracle/_ref/ (oracle/build_ref.py)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def dev():
    if not torch.cuda.is_available():
        pytest.skip('needs a CUDA device')
    return torch.device('cuda:0')


@pytest.fixture(scope='module')
def ref(dev):
    from oracle.ref_pipeline import load_reference
    r = load_reference()
    if r is None:
        pytest.skip('oracle/_ref is not staged (python oracle/build_ref.py --ref <reference checkout>)')
    return r


def same(a, b, what):
    if isinstance(a, torch.Tensor):
        assert isinstance(b, torch.Tensor) and a.shape == b.shape and a.dtype == b.dtype, f'{what}: {a.shape} {a.dtype} vs {getattr(b, "shape", None)} {getattr(b, "dtype", None)}'
        assert torch.equal(a, b), f'{what} differs'
    else:
        assert a == b, f'{what}: {a} vs {b}'


PLAN_TENSORS = ('u', 'hit_pos', 'hit_slot', 'N_pos', 'N_row', 'L_pos', 'L_row', 'L_cnt', 'F_pos', 'F_row', 'S_pos', 'S_row', 'L_steps',
                'ev_slot', 'ev_row', 'ev_rep', 'L_off', 'adm_rec_dyn', 'evM_slot', 'evl_src')
# outputs whose entries for slots that record nothing point at the trash row: compared where they are meaningful
STATE = ('code', 'adm_c0', 'rj', 'rok', 'kthr', 'toff', 'slot_of', 'slot_row', 'n_lfree', 'log_top', 'mat_top', 'live', 'free', 'dyn_slots',
         'tcount', 'last_seen', 'pinned')


@pytest.mark.parametrize('R,C,dyn_slots,batch,steps,dyn,st_mode,expect', [
    (2_000_000, 200_000, 32_768, 2048, 40, 'ttl', 'T', ()),
    (20_000, 1_200, 200, 96, 40, 'ttl', 'T', ('preempt', 'overflow')),
    (20_000, 1_100, 100, 96, 40, 'carry', 'S', ('overflow',)),
    (20_000, 1_020, 20, 128, 40, 'ttl', 'S', ('preempt', 'overflow')),
])
def test_plan_equals_the_reference_planner(dev, ref, R, C, dyn_slots, batch, steps, dyn, st_mode, expect):
    from elara_b200 import synth, planner
    from elara_b200.ops import dir_ext
    relara = ref['elara']
    K, L, depth, seed = 3, 4, 3, 3
    sizes, offs = synth.table_sizes(R, 26, lo=4, hi=max(8, R // 4), seed=seed)
    ids = [torch.from_numpy(synth.zipf_lookups(sizes, offs, batch, 1.1, seed, s + 1)).to(dev) for s in range(steps)]
    U = [torch.unique(i) for i in ids]
    uu, cc = torch.unique(torch.cat(ids[:4]), return_counts=True)
    n0 = min(C - dyn_slots, uu.numel())
    static = uu[torch.argsort(cc, descending=True, stable=True)[:n0]].sort().values

    def make():
        pl = relara.ELARAPlanner(R, C, K, 'static', dyn, st_mode, static, L, dev, torch.from_numpy(offs), torch.full((26,), K, dtype=torch.int8),
                                 evict_logs=1, dir_impl='cpp')
        pl.code[static] = pl.MAT
        return pl
    a, b = make(), make()
    b.dx = dir_ext()
    for j in range(min(steps, L + 1)):
        a.observe(j + 1, U[j]); b.observe(j + 1, U[j])
    for s in range(steps):
        if s + L + 1 < steps:
            a.observe(s + L + 2, U[s + L + 1]); b.observe(s + L + 2, U[s + L + 1])
        nexts = [U[s + k] for k in range(1, depth) if s + k < steps]
        pa = a.plan(s + 1, U[s], nexts)
        pb = planner.plan(b, s + 1, U[s], nexts)
        for k in ('s', 'n', 'barrier', 'evl'):
            same(getattr(pa, k), getattr(pb, k), f'step {s + 1} {k}')
        for k in PLAN_TENSORS:
            same(getattr(pa, k), getattr(pb, k), f'step {s + 1} {k}')
        # history slots of hits that record nothing and of evicted slots' dyn index: identical by construction as well
        same(pa.hrec_dyn, pb.hrec_dyn, f'step {s + 1} hrec_dyn'); same(pa.hrec_j, pb.hrec_j, f'step {s + 1} hrec_j')
        same(pa.ev_dyn, pb.ev_dyn, f'step {s + 1} ev_dyn')
        assert set(pa.ix) == set(pb.ix)
        for k in pa.ix:
            same(pa.ix[k], pb.ix[k], f'step {s + 1} ix[{k}]')
        assert set(pa.cpu) == set(pb.cpu)
        for k in pa.cpu:
            same(pa.cpu[k], pb.cpu[k], f'step {s + 1} cpu[{k}]')
    torch.cuda.synchronize()
    for k in STATE:
        same(getattr(a, k), getattr(b, k), f'planner.{k}')
    Kk, nf = a.Kmax, int(a.n_lfree)
    same(a.loc[:R], b.loc[:R], 'loc'); same(a.ent[:R * Kk], b.ent[:R * Kk], 'ent'); same(a.lstep[:a.log_cap], b.lstep[:a.log_cap], 'lstep')
    same(a.lfree[:nf], b.lfree[:nf], 'lfree'); same(a.pstep[:a.Cdyn], b.pstep[:a.Cdyn], 'pstep')
    sa = {k: v for k, v in a.stats.items() if k != 'syncs'}
    sb = {k: v for k, v in b.stats.items() if k != 'syncs'}
    assert sa == sb
    assert b.stats['syncs'] <= a.stats['syncs']
    for k in expect:
        assert a.stats.get(k, 0) > 0, f'{k} never ran in this configuration'
