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
