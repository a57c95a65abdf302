"""Planner classification + class partition (srm2_plan_classify) against the reference planner's recorded plans
(tests/golden/plan_*.npz) and against the NumPy oracle on a large random case."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def dev():
    assert torch.cuda.is_available(), 'these tests need a CUDA device'
    from elara_b200 import _lib
    _lib.lib()
    return torch.device('cuda:0')


def run(dev, u, nexts, slot_of, last_seen, code, kthr, toff, s, K, ttl, want_T, admit=None):
    from elara_b200.planner import plan_classify
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    r = plan_classify(t(u), [t(x) for x in nexts], t(slot_of), t(last_seen), t(code), t(kthr), t(toff), s, K, ttl, want_T,
                      admit=None if admit is None else t(admit))
    torch.cuda.synchronize()
    return {k: getattr(r, k).cpu().numpy() for k in ('sl', 'in_next', 'admit', 'c', 'cls', 'counts', 'order', 'bad_rows')}


def same(got, want):
    for k in ('sl', 'in_next', 'admit', 'c', 'cls', 'counts', 'order'):
        assert np.array_equal(got[k], want[k]), k
    assert int(got['bad_rows'][0]) == 0


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_plan_classify_vs_reference_planner(dev, oracle, golden_dir, name):
    from test_oracle_golden import plan_golden_steps
    for g, s, nexts in plan_golden_steps(golden_dir, name):
        a = (g[f's{s}_u'], nexts, g[f's{s}_slot_of'], g[f's{s}_last_seen'], g[f's{s}_code'], g['kthr'], g['toff'], s, int(g['K']), int(g['ttl']),
             int(g['want_T']))
        got = run(dev, *a)
        same(got, oracle.plan_classify(*a))
        pos = oracle.plan_positions(got)
        for k, v in pos.items():
            assert np.array_equal(v, g[f's{s}_{k}']), (name, s, k)          # the reference's own position lists
        assert np.array_equal(got['sl'][pos['hit_pos']].astype(np.int64), g[f's{s}_hit_slot'])


@pytest.mark.parametrize('n,ttl,want_T,n_lists', [(50_000, 1, 1, 2), (50_000, 0, 0, 3), (1, 1, 0, 0), (1025, 0, 1, 8), (0, 1, 1, 1)])
def test_plan_classify_vs_oracle_large(dev, oracle, n, ttl, want_T, n_lists):
    rng = np.random.default_rng(n + ttl + 7 * n_lists)
    R, C, K, T = 1_000_000, 200_000, 3, 26
    toff = np.concatenate([[0], np.sort(rng.choice(np.arange(1, R), size=T - 1, replace=False))]).astype(np.int64)
    kthr = rng.integers(0, K + 1, size=T).astype(np.int8)
    code = rng.choice(np.arange(0, K + 2), size=R, p=(.5, .15, .1, .05, .2)).astype(np.int8)
    slot_of = np.full(R, -1, np.int32)
    res = rng.choice(R, size=C, replace=False); slot_of[res] = rng.permutation(C).astype(np.int32)
    last_seen = rng.integers(-1, 60, size=R).astype(np.int32)
    u = np.sort(rng.choice(R, size=n, replace=False)).astype(np.int64)
    nexts = [np.sort(rng.choice(R, size=int(rng.integers(1, 60_000)), replace=False)).astype(np.int64) for _ in range(n_lists)]
    if n_lists and n:
        nexts[0][: min(len(nexts[0]), n // 2 + 1)] = np.sort(u[: min(len(nexts[0]), n // 2 + 1)])   # real overlap with u
        nexts[0] = np.unique(nexts[0])
    a = (u, nexts, slot_of, last_seen, code, kthr, toff, 30, K, ttl, want_T)
    want = oracle.plan_classify(*a)
    got = run(dev, *a)
    same(got, want)
    if n:      # the second classification of the reference: a given admission mask
        adm = want['admit'] & (rng.random(n) < 0.5)
        same(run(dev, *a, admit=adm), oracle.plan_classify(*a, admit=adm))


def test_plan_classify_counts_bad_rows(dev):
    """Row ids outside the directory are counted and classified C_S without any read."""
    z32 = np.full(10, -1, np.int32)
    got = run(dev, np.array([-5, 3, 10, 99], np.int64), [], z32, z32, np.zeros(10, np.int8), np.array([1], np.int8), np.array([0], np.int64), 1, 3, 1, 1)
    assert int(got['bad_rows'][0]) == 3 and got['cls'].tolist() == [9, 2, 9, 9] and int(got['counts'].sum()) == 1


def run_ev(dev, nexts, slot_of, pinned, dyn_slots, slot_row, last_seen, s, ttl):
    from elara_b200.planner import evict_candidates
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    r = evict_candidates([t(x) for x in nexts], t(slot_of), t(pinned), t(dyn_slots), t(slot_row), t(last_seen), s, ttl)
    torch.cuda.synchronize()
    n_exp = int(r.n_exp.item()); parted = r.parted.cpu().numpy()
    return dict(protect=r.protect.cpu().numpy(), exp=r.exp.cpu().numpy(), n_exp=n_exp, ev_slot=parted[:n_exp], keep_dyn=parted[n_exp:])


def same_ev(got, want):
    assert got['n_exp'] == want['n_exp']
    for k in ('protect', 'exp', 'ev_slot', 'keep_dyn'):
        assert np.array_equal(got[k], want[k]), k


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_evict_candidates_vs_reference_planner(dev, oracle, golden_dir, name):
    from test_oracle_golden import plan_golden_steps
    for g, s, nexts in plan_golden_steps(golden_dir, name):
        a = (nexts, g[f's{s}_slot_of'], g[f's{s}_pinned'], g[f's{s}_dyn_slots'], g[f's{s}_slot_row'], g[f's{s}_last_seen'], s, int(g['ttl']))
        got = run_ev(dev, *a)
        same_ev(got, oracle.plan_evict_candidates(*a))
        if s == 1 or int(g[f's{s}_preempt']) == int(g[f's{s - 1}_preempt']):
            assert np.array_equal(got['ev_slot'], g[f's{s}_ev_slot']), (name, s)                 # the reference's own choice
            assert np.array_equal(got['keep_dyn'], g[f's{s}_dyn_slots_after'][:len(got['keep_dyn'])]), (name, s)


@pytest.mark.parametrize('nd,ttl,n_lists', [(131_072, 1, 2), (131_072, 0, 3), (5, 1, 0), (0, 1, 1), (2_000_000, 1, 2)])
def test_evict_candidates_vs_oracle_large(dev, oracle, nd, ttl, n_lists):
    rng = np.random.default_rng(nd + ttl + n_lists)
    R, C = 4_000_000, max(2 * nd, 1000)
    n0 = C - nd
    slot_row = np.full(C, -1, np.int64); slot_of = np.full(R, -1, np.int32)
    rows = rng.choice(R, size=C, replace=False).astype(np.int64)
    slot_row[:] = rows; slot_of[rows] = np.arange(C, dtype=np.int32)
    pinned = np.zeros(C, bool); pinned[:n0] = True
    dyn_slots = (n0 + rng.permutation(nd)).astype(np.int64)
    last_seen = rng.integers(-1, 60, size=R).astype(np.int32)
    nexts = [np.sort(np.concatenate([rng.choice(rows, size=min(C, 20_000), replace=False), rng.choice(R, size=5000)])).astype(np.int64)
             for _ in range(n_lists)]
    nexts = [np.unique(x) for x in nexts]
    a = (nexts, slot_of, pinned, dyn_slots, slot_row, last_seen, 30, ttl)
    same_ev(run_ev(dev, *a), oracle.plan_evict_candidates(*a))


def run_pack(dev, ev_slot, rep, evf_slots, evl_ids, ev_dyn, K, loc, F_row, S_row, nFa, c_slots, L_ids, a_ids, tops3):
    from elara_b200.planner import pack
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    top = [torch.tensor([int(v)], dtype=torch.int64, device=dev) for v in tops3]
    r = pack(t(ev_slot), t(rep), t(evf_slots), t(evl_ids), t(ev_dyn), K, t(loc), t(F_row), t(S_row), nFa, t(c_slots), t(L_ids), t(a_ids), *top)
    torch.cuda.synchronize()
    flat = r.flat.cpu().numpy(); out = dict(evM_slot=r.evM_slot.cpu().numpy(), evl_src=r.evl_src.cpu().numpy()); o = 0
    for name, n in r.parts:
        out[name] = flat[o:o + n]; o += n
    assert o == len(flat)
    return out


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_plan_pack_vs_reference_planner(dev, oracle, golden_dir, name):
    from test_oracle_golden import plan_golden_steps, plan_pack_args
    for g, s, _ in plan_golden_steps(golden_dir, name):
        got = run_pack(dev, *plan_pack_args(g, s))
        assert np.array_equal(got['evM_slot'], g[f's{s}_pk_evM_slot']) and np.array_equal(got['evl_src'], g[f's{s}_pk_evl_src']), (name, s)
        for k in ('S_slot', 'F_slot', 'L_ids', 'A_ids', 'W_slot', 'EVL_ids', 'tops'):
            assert np.array_equal(got[k], g[f's{s}_pk_cpu_{k}']), (name, s, k)            # the reference's own host lists


@pytest.mark.parametrize('nev,K,nF,nS', [(40_000, 3, 3000, 2000), (1, 1, 0, 0), (0, 3, 10, 7), (5000, 5, 0, 1)])
def test_plan_pack_vs_oracle_large(dev, oracle, nev, K, nF, nS):
    rng = np.random.default_rng(nev + K + nF)
    R = 2_000_000
    loc = rng.integers(-1, 1 << 20, size=R + 1).astype(np.int32)
    ev_slot = rng.permutation(1 << 20)[:nev].astype(np.int64)
    rep = rng.random(nev) < 0.4
    evf_slots = rng.integers(0, 1 << 22, size=nev).astype(np.int64)
    evl_ids = np.where(rng.random((nev, K)) < 0.5, rng.integers(0, 1 << 24, size=(nev, K)), -1).astype(np.int64)
    ev_dyn = rng.permutation(1 << 18)[:nev].astype(np.int64) if nev <= (1 << 18) else rng.integers(0, 1 << 18, size=nev).astype(np.int64)
    F_row = rng.choice(R, size=nF, replace=False).astype(np.int64); S_row = rng.choice(R, size=nS, replace=False).astype(np.int64)
    nFa = nF // 3
    c_slots = rng.integers(0, 1 << 22, size=777 if nev else 0).astype(np.int64)
    L_ids = rng.integers(-1, 1 << 24, size=(1234 if nev else 2, K)).astype(np.int32)
    a_ids = rng.integers(0, 1 << 24, size=4321 if nev else 0).astype(np.int64)
    a = (ev_slot, rep, evf_slots, evl_ids, ev_dyn, K, loc, F_row, S_row, nFa, c_slots, L_ids, a_ids, np.array([11, 22, 33]))
    want = oracle.plan_pack(*a)
    got = run_pack(dev, *a)
    for k in want:
        assert np.array_equal(got[k], want[k]), k
