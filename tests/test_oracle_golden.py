"""The CPU oracle against the golden vectors produced by the reference itself (tests/golden/make_golden.py)
and, where the compiled reference sources are present (oracle/_ref), against the reference directly."""
import zlib

import numpy as np
import pytest


def eq_bits(a, b):
    a = np.ascontiguousarray(a); b = np.ascontiguousarray(b)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_adam_scalars(oracle, golden_dir):
    g = np.load(golden_dir / 'adam_scalars.npz')
    for h, row in zip(g['hyper'], g['scalars']):
        for s, want in zip(g['steps'], row):
            assert eq_bits(oracle.adam_scalars(*h, int(s)), want)


@pytest.mark.parametrize('name', ['adam_d16', 'adam_d24', 'adam_d128'])
def test_adam_rows(oracle, golden_dir, name):
    g = np.load(golden_dir / f'{name}.npz')
    st = g['state0'].copy()
    h = g['hyper']
    for rows, grad, t, sc in zip(g['rows'], g['grad'], g['steps'], g['scalars']):
        assert eq_bits(oracle.adam_scalars(*h, int(t)), sc)
        oracle.adam_rows(st, rows, np.ascontiguousarray(grad), *h, int(t), nthreads=3)
    assert eq_bits(st, g['state_out'])


def test_init_rows(oracle, golden_dir):
    g = np.load(golden_dir / 'init_rows.npz')
    rows = g['rows']
    keys = [k for k in g.files if k.startswith('D') and not k.endswith('_bound')]
    assert len(keys) == 20
    for k in keys:
        D = int(k[1:].split('_')[0]); seed = int(k.split('seed')[1])
        out = oracle.init_rows(rows, D, seed, float(g[k + '_bound']))
        assert eq_bits(out, g[k]), k
        assert np.all(out[:, 1:] == 0)


@pytest.mark.parametrize('name', ['replay_d64_k3', 'replay_d128_k3', 'replay_d24_k2', 'replay_d16_k4'])
def test_replay_rows(oracle, golden_dir, name):
    g = np.load(golden_dir / f'{name}.npz')
    D, K, seed, smax = (int(x) for x in g['meta'])
    table = oracle.scalar_table(*g['hyper'], smax)
    assert eq_bits(table, g['table'])
    out = oracle.replay_rows(g['rows'], g['logs'], g['offs'], g['steps'], g['cnt'], D, K, seed, float(g['bound']), table)
    assert eq_bits(out, g['out'])
    assert (g['cnt'] == 0).any() and (g['cnt'] == K).any()


def test_unique_inverse(oracle):
    rng = np.random.default_rng(0)
    for n in (0, 1, 7, 1000):
        ids = rng.integers(0, 50, n).astype(np.int64) * 10**9
        u, inv = oracle.unique_inverse(ids)
        ur, invr = np.unique(ids, return_inverse=True)
        assert np.array_equal(u, ur) and np.array_equal(inv, invr.reshape(-1))


def test_segment_reduce_orders(oracle):
    """Both summation orders give the exact sum on values where fp32 addition is exact, and the chunked
    order differs from the left-to-right one where it must (mixed magnitudes)."""
    rng = np.random.default_rng(1)
    inv = rng.integers(0, 5, 200).astype(np.int64)
    grad = rng.integers(-8, 8, (200, 4)).astype(np.float32)
    want = np.zeros((5, 4), np.float32)
    np.add.at(want, inv, grad)
    assert np.array_equal(oracle.segment_reduce(grad, inv, 5, chunk=10), want)
    assert np.array_equal(oracle.segment_reduce(grad, inv, 5, chunk=0), want)
    g2 = np.array([[1e8]] + [[1.0]] * 19, np.float32); i2 = np.zeros(20, np.int64)
    seq = oracle.segment_reduce(g2, i2, 1, chunk=0); chk = oracle.segment_reduce(g2, i2, 1, chunk=10)
    assert seq[0, 0] == np.float32(1e8) and chk[0, 0] == np.float32(1e8) + np.float32(10.0)


def test_segment_reduce_golden(oracle, golden_dir):
    """Vectors produced on a B200 by PyTorch's CUDA aten.embedding_dense_backward (tests/golden/make_segreduce_golden.py);
    cases where that operator's default mode is not run-to-run deterministic hold its deterministic-mode output."""
    g = np.load(golden_dir / 'segreduce_cuda.npz')
    assert str(g['torch_version']).startswith('2.11')
    small = large = unstable = 0
    for ci in range(int(g['n_cases'])):
        grad, inv, nu = g[f'c{ci}_grad'], g[f'c{ci}_inv'], int(g[f'c{ci}_nu'])
        assert eq_bits(oracle.segment_reduce(grad, inv, nu), g[f'c{ci}_out']), ci
        small += len(inv) <= 3072; large += len(inv) > 3072; unstable += not bool(g[f'c{ci}_default_mode_stable'])
    assert small > 10 and large > 5 and unstable > 0


DIR_OUT_A = ('L_steps', 'L_ids', 'hrec_dyn', 'hrec_j', 'ev_row', 'rep', 'evl_ids', 'evf_slots', 'ev_dyn')


def run_dir_trace(O, g, make_dir, check_state):
    """Replay a recorded planner trace through a directory implementation (oracle or CUDA)."""
    pvk = ('R', 'K', 'Lcap', 'n0', 'Cdyn', 'MAT', 'trash', 'evl')
    pv = dict(zip(pvk, (int(x) for x in g['pv'])))
    st0 = {k: g[f'init_{k}'] for k in O.DIR_FIELDS}
    d = make_dir(st0, pv)
    n_rep = n_evl = 0
    for s in range(1, int(g['steps']) + 1):
        o = d.dir_a(g[f's{s}_hs'], g[f's{s}_L_row'], g[f's{s}_L_cnt'], g[f's{s}_ev_slot'], s)
        for k in DIR_OUT_A:
            want = g[f's{s}_o_{k}']
            got = np.asarray(o[k]).reshape(want.shape)
            if k == 'evl_ids' or k == 'rep':
                got = got.astype(want.dtype)
            assert np.array_equal(got, want), (s, k)
        n_rep += int(g[f's{s}_o_rep'].sum()); n_evl += int((g[f's{s}_o_evl_ids'] >= 0).sum())
        check_state(d, pv, g[f's{s}_crc'][0], (s, 'a'))
        d.admit(g[f's{s}_adm_rows'], g[f's{s}_adm_slots'], int(g[f's{s}_lazy_n']), s)
        check_state(d, pv, g[f's{s}_crc'][1], (s, 'adm'))
        o = d.dir_b(g[f's{s}_a_rows'], g[f's{s}_a_k'], g[f's{s}_c_rows'], g[f's{s}_c_cnt'], s)
        assert np.array_equal(np.asarray(o['a_ids']), g[f's{s}_o_a_ids']), (s, 'a_ids')
        assert np.array_equal(np.asarray(o['c_slots']), g[f's{s}_o_c_slots']), (s, 'c_slots')
        check_state(d, pv, g[f's{s}_crc'][2], (s, 'b'))
        if f's{s}_state_code' in g.files:
            cur = O.dir_comparable(d.state(), pv)
            want = O.dir_comparable({k: (g[f's{s}_state_{k}'] if f's{s}_state_{k}' in g.files else st0[k]) for k in O.DIR_FIELDS}, pv)
            for k in O.DIR_FIELDS:
                assert np.array_equal(cur[k].reshape(-1), want[k].reshape(-1)), (s, k)
    return n_rep, n_evl


def crc_check(O):
    def check(d, pv, want, where):
        cmp = O.dir_comparable(d.state(), pv)
        got = np.array([zlib.crc32(np.ascontiguousarray(cmp[k]).tobytes()) for k in O.DIR_FIELDS], np.int64)
        bad = [k for k, a, b in zip(O.DIR_FIELDS, got, want) if a != b]
        assert not bad, (where, bad)
    return check


@pytest.mark.parametrize('name', ['dir_ttl_evl1', 'dir_ttl_evl0', 'dir_carry_evl1'])
def test_directory_trace(oracle, golden_dir, name):
    g = np.load(golden_dir / f'{name}.npz')

    class D(oracle.Directory):
        def state(self):
            return self.st
    n_rep, n_evl = run_dir_trace(oracle, g, lambda st, pv: D(st, pv), crc_check(oracle))
    if name.endswith('evl1'):
        assert n_rep > 0 and n_evl > 0          # the trace exercises evictions back to the logged state


def test_oracle_vs_compiled_reference(oracle):
    """Larger random cases against the reference's own C++ (skipped where oracle/_ref was not built)."""
    E = oracle.ref_cpu()
    if E is None:
        pytest.skip('compiled reference sources not present')
    import torch
    rng = np.random.default_rng(5)
    for D in (16, 40, 128):
        R, n = 20000, 6000
        st = (rng.standard_normal((R, 3, D)) * 0.05).astype(np.float32); st[:, 1:] = 0
        ref = torch.from_numpy(st.copy())
        for step in range(1, 5):
            rows = np.sort(rng.choice(R, n, replace=False)).astype(np.int64)
            grad = (rng.standard_normal((n, D)) * 10.0 ** (step % 3 - 2)).astype(np.float32)
            oracle.adam_rows(st, rows, grad, 1e-3, 0.9, 0.999, 1e-8, step, nthreads=4)
            E.cpu_adam(ref, torch.from_numpy(rows), torch.from_numpy(grad), 1e-3, 0.9, 0.999, 1e-8, step, 8)
        assert eq_bits(st, ref.numpy())


def plan_golden_steps(golden_dir, name):
    g = np.load(golden_dir / f'{name}.npz')
    for s in range(1, int(g['steps']) + 1):
        if int(g[f's{s}_overflow']):
            continue
        nexts = [g[f's{s}_next{q}'] for q in range(int(g[f's{s}_n_next']))]
        yield g, s, nexts


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_plan_classify_oracle_vs_reference_planner(oracle, golden_dir, name):
    """The NumPy restatement of the planner's classification reproduces the position lists the reference's own
    ELARAPlanner.plan returned (tests/golden/make_plan_golden.py)."""
    seen = set()
    for g, s, nexts in plan_golden_steps(golden_dir, name):
        r = oracle.plan_classify(g[f's{s}_u'], nexts, g[f's{s}_slot_of'], g[f's{s}_last_seen'], g[f's{s}_code'], g['kthr'], g['toff'], s,
                                 int(g['K']), int(g['ttl']), int(g['want_T']))
        pos = oracle.plan_positions(r)
        for k, v in pos.items():
            assert np.array_equal(v, g[f's{s}_{k}']), (name, s, k)
        assert np.array_equal(r['sl'][pos['hit_pos']].astype(np.int64), g[f's{s}_hit_slot'])
        assert np.array_equal(r['c'][pos['L_pos']].astype(np.int32), g[f's{s}_L_cnt'])
        assert int(r['counts'][oracle.C_NADM]) == int(g[f's{s}_N_n_adm']) and int(r['counts'][oracle.C_LADM]) == int(g[f's{s}_L_n_adm'])
        seen |= set(np.flatnonzero(r['counts']).tolist())
    assert len(seen) >= 8          # the traces exercise nearly every class


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_plan_evict_candidates_oracle_vs_reference_planner(oracle, golden_dir, name):
    """Eviction candidates and surviving dynamic slots as the reference planner chose them (steps without preemption)."""
    n_ev = 0
    for g, s, nexts in plan_golden_steps(golden_dir, name):
        if s > 1 and int(g[f's{s}_preempt']) != int(g[f's{s - 1}_preempt']):
            continue
        r = oracle.plan_evict_candidates(nexts, g[f's{s}_slot_of'], g[f's{s}_pinned'], g[f's{s}_dyn_slots'], g[f's{s}_slot_row'], g[f's{s}_last_seen'],
                                         s, int(g['ttl']))
        assert np.array_equal(r['ev_slot'], g[f's{s}_ev_slot']), (name, s)
        assert np.array_equal(r['keep_dyn'], g[f's{s}_dyn_slots_after'][:len(r['keep_dyn'])]), (name, s)
        n_ev += r['n_exp']
    assert n_ev > 50


def plan_pack_args(g, s):
    return (g[f's{s}_ev_slot'], g[f's{s}_pk_rep'], g[f's{s}_pk_evf_slots'], g[f's{s}_pk_evl_ids'], g[f's{s}_pk_ev_dyn'], int(g['K']), g[f's{s}_pk_loc'],
            g[f's{s}_pk_F_row'], g[f's{s}_pk_S_row'], int(g[f's{s}_pk_nFa']), g[f's{s}_pk_c_slots'], g[f's{s}_pk_L_ids'], g[f's{s}_pk_a_ids'],
            g[f's{s}_pk_tops'])


@pytest.mark.parametrize('name', ['plan_ttl_T', 'plan_carry_S'])
def test_plan_pack_oracle_vs_reference_planner(oracle, golden_dir, name):
    """Packed eviction outputs and host work lists exactly as the reference planner returned them."""
    n = 0
    for g, s, _ in plan_golden_steps(golden_dir, name):
        r = oracle.plan_pack(*plan_pack_args(g, s))
        assert np.array_equal(r['evM_slot'], g[f's{s}_pk_evM_slot']) and np.array_equal(r['evl_src'], g[f's{s}_pk_evl_src']), (name, s)
        for k in ('S_slot', 'F_slot', 'L_ids', 'A_ids', 'W_slot', 'EVL_ids', 'tops'):
            assert np.array_equal(r[k], g[f's{s}_pk_cpu_{k}']), (name, s, k)
        n += len(r['W_slot'])
    assert n > 100
