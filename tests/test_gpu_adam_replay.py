"""Bitwise parity of the CUDA Adam / init / replay kernels (called through the C ABI via the srm2-style Python
mirror) with the CPU oracle, the golden vectors of the reference, and size-independent properties at full size."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.fixture(scope='module')
def dev():
    assert torch.cuda.is_available(), 'these tests need a CUDA device'
    from elara_b200 import _lib
    _lib.lib()
    return torch.device('cuda:0')


# ------------------------------------------------------------------------------------------------ Adam
@pytest.mark.parametrize('name', ['adam_d16', 'adam_d24', 'adam_d128'])
def test_adam_golden(dev, golden_dir, name):
    from elara_b200.ops import gpu_adam
    g = np.load(golden_dir / f'{name}.npz')
    pool = torch.from_numpy(g['state0'].copy()).to(dev)
    for k, (rows, grad, t) in enumerate(zip(g['rows'], g['grad'], g['steps'])):
        r = torch.from_numpy(rows).to(dev)
        gpu_adam(pool, r.to(torch.int32) if k % 2 else r, torch.from_numpy(grad).to(dev), *g['hyper'], int(t))
    assert np.array_equal(bits(pool.cpu().numpy()), bits(g['state_out']))


@pytest.mark.parametrize('D', [16, 24, 40, 64, 128, 7, 1, 130])
def test_adam_vs_oracle(dev, oracle, D):
    from elara_b200.ops import gpu_adam
    rng = np.random.default_rng(D)
    R, n = 5000, 1777
    st = (rng.standard_normal((R, 3, D)) * 0.05).astype(np.float32); st[:, 1:] = 0
    pool = torch.from_numpy(st.copy()).to(dev)
    for step in range(1, 6):
        rows = rng.choice(R, n, replace=False).astype(np.int64)
        if step % 2:
            rows.sort()
        grad = (rng.standard_normal((n, D)) * 10.0 ** (step % 3 - 2)).astype(np.float32)
        if step == 4:
            grad[:50] = 0; grad[50:60] = 1e-30; grad[60:70] = -0.0; grad[70:80] = 3e4
        oracle.adam_rows(st, rows, grad, *HYP, step * 13)
        r = torch.from_numpy(rows).to(dev)
        gpu_adam(pool, r if step % 3 else r.to(torch.int32), torch.from_numpy(grad).to(dev), *HYP, step * 13)
    assert np.array_equal(bits(pool.cpu().numpy()), bits(st))


def test_adam_unaligned_views_and_empty(dev, oracle):
    from elara_b200.ops import gpu_adam
    rng = np.random.default_rng(3)
    R, D, n = 300, 16, 64
    st = (rng.standard_normal((R, 3, D)) * 0.05).astype(np.float32); st[:, 2] = np.abs(st[:, 2])
    # gradient matrix that starts 4 bytes into its storage: not 16-byte aligned
    flat = torch.zeros(n * D + 1, device=dev)
    grad = (rng.standard_normal((n, D)) * 1e-2).astype(np.float32)
    flat[1:] = torch.from_numpy(grad).to(dev).reshape(-1)
    gview = flat[1:].view(n, D)
    rows = rng.choice(R, n, replace=False).astype(np.int64)
    pool = torch.from_numpy(st.copy()).to(dev)
    gpu_adam(pool, torch.from_numpy(rows).to(dev), gview, *HYP, 3)
    oracle.adam_rows(st, rows, grad, *HYP, 3)
    assert np.array_equal(bits(pool.cpu().numpy()), bits(st))
    before = pool.clone()
    gpu_adam(pool, torch.empty(0, dtype=torch.int64, device=dev), torch.empty(0, D, device=dev), *HYP, 4)
    assert torch.equal(pool, before)


def test_adam_reference_test_shapes(dev, oracle):
    """Shapes of the reference's own exactness test (tests/test_ops.py:11-24): R=200,000, D=128, 6 steps of
    30,000 sorted distinct rows, gradient scale 10^(step%3-2)."""
    from elara_b200.ops import gpu_adam
    g0 = torch.Generator().manual_seed(0)
    R, D = 200_000, 128
    host = torch.randn(R, 3, D, generator=g0) * 0.05; host[:, 1:] = 0
    gpu = host.clone().to(dev); st = host.numpy()
    for step in range(1, 7):
        rows = torch.randperm(R, generator=g0)[:30000].sort().values
        grad = torch.randn(len(rows), D, generator=g0) * (10.0 ** (step % 3 - 2))
        oracle.adam_rows(st, rows.numpy(), grad.numpy(), *HYP, step, nthreads=8)
        gpu_adam(gpu, rows.to(dev), grad.to(dev), *HYP, step)
    assert np.array_equal(bits(gpu.cpu().numpy()), bits(st))


def test_adam_config1_100_steps(dev, oracle):
    """1,000,000 x 16 table, 100 steps of 65,536 distinct Zipf(1.05) rows, bitwise against the oracle."""
    from elara_b200 import synth
    from elara_b200.ops import gpu_adam
    from elara_b200.gpu_ops import init_rows
    R, D, n = 1_000_000, 16, 65_536
    pool = init_rows(torch.arange(R, device=dev), D, 42, 0.01)
    st = pool.cpu().numpy().copy()
    assert np.array_equal(bits(st), bits(oracle.init_rows(np.arange(R), D, 42, 0.01)))
    for step in range(1, 101):
        rows = synth.zipf_rows_without_replacement(R, n, 1.05, 42, step, sort=(step % 10 != 0))
        grad = synth.normal_f32((n, D), 1e-3, 42, step)
        oracle.adam_rows(st, rows, grad, *HYP, step, nthreads=8)
        gpu_adam(pool, torch.from_numpy(rows).to(dev), torch.from_numpy(grad).to(dev), *HYP, step)
    assert np.array_equal(bits(pool.cpu().numpy()), bits(st))


# ------------------------------------------------------------------------------------------------ init
def test_init_golden(dev, golden_dir):
    from elara_b200.gpu_ops import init_rows
    g = np.load(golden_dir / 'init_rows.npz')
    rows = torch.from_numpy(g['rows']).to(dev)
    for k in [k for k in g.files if k.startswith('D') and not k.endswith('_bound')]:
        D = int(k[1:].split('_')[0]); seed = int(k.split('seed')[1])
        out = init_rows(rows, D, seed, float(g[k + '_bound']))
        assert np.array_equal(bits(out.cpu().numpy()), bits(g[k])), k


@pytest.mark.parametrize('D', [16, 24, 64, 128, 5, 132])
def test_init_vs_oracle_and_permutation(dev, oracle, D):
    from elara_b200.gpu_ops import init_rows
    rng = np.random.default_rng(D)
    rows = np.unique(np.concatenate([rng.integers(0, 30_000_000, 3000), rng.integers(2**31 - 5, 2**31 + 5, 10),
                                     rng.integers(2**32 - 5, 2**32 + 5, 10), rng.integers(2**40, 2**41, 10)])).astype(np.int64)
    r = torch.from_numpy(rows).to(dev)
    a = init_rows(r, D, 1234, 0.01)
    assert np.array_equal(bits(a.cpu().numpy()), bits(oracle.init_rows(rows, D, 1234, 0.01)))
    perm = torch.randperm(len(rows), device=dev)
    b = init_rows(r[perm], D, 1234, 0.01)            # determinism check of tests/test_replay.py:17-18
    assert torch.equal(a[perm], b)
    out = torch.full((len(rows), 3, D), 7.0, device=dev)
    assert init_rows(r, D, 1234, 0.01, out=out) is out and torch.equal(out, a)
    assert init_rows(torch.empty(0, dtype=torch.int64, device=dev), D, 1, 0.1).shape == (0, 3, D)


# ---------------------------------------------------------------------------------------------- replay
@pytest.mark.parametrize('name', ['replay_d64_k3', 'replay_d128_k3', 'replay_d24_k2', 'replay_d16_k4'])
def test_replay_golden(dev, golden_dir, name):
    from elara_b200.gpu_ops import replay_rows, ScalarTable
    g = np.load(golden_dir / f'{name}.npz')
    D, K, seed, smax = (int(x) for x in g['meta'])
    table = ScalarTable(*g['hyper'], smax, dev)
    assert np.array_equal(bits(table.t.cpu().numpy()), bits(g['table']))
    t = lambda k: torch.from_numpy(g[k]).to(dev)
    out = replay_rows(t('rows'), t('logs'), t('offs'), t('steps'), t('cnt'), D, K, seed, float(g['bound']), table)
    assert np.array_equal(bits(out.cpu().numpy()), bits(g['out']))


@pytest.mark.parametrize('D,K', [(64, 3), (128, 3), (16, 1), (24, 2), (64, 5), (32, 9), (6, 3), (64, 0)])
def test_replay_vs_oracle(dev, oracle, D, K):
    from elara_b200 import synth
    from elara_b200.gpu_ops import replay_rows, ScalarTable
    n = 4000
    c = synth.replay_case(n, 4_000_000, D, max(K, 1), 50, 100 + D + K, min_cnt=0)
    if K == 0:
        c['cnt'][:] = 0; c['steps'] = np.zeros((n, 0), np.int32); c['logs'] = np.zeros((0, D), np.float32); c['offs'][:] = 0
    c['rows'][-1] = 2**33 + 5
    table = ScalarTable(*HYP, 50, dev)
    t = lambda k: torch.from_numpy(c[k]).to(dev)
    out = replay_rows(t('rows'), t('logs'), t('offs'), t('steps'), t('cnt'), D, K, 1234, 0.01, table)
    want = oracle.replay_rows(c['rows'], c['logs'], c['offs'], c['steps'], c['cnt'], D, K, 1234, 0.01, oracle.scalar_table(*HYP, 50))
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))
    assert (c['cnt'] == 0).any()          # rows without history come back as the pure initialisation


def test_replay_config2_full_size(dev, oracle):
    """262,144 rows x 64, histories of 1..3 gradients at steps in [1,50]: replay equals eager Adam applied at
    those steps (the construction of the reference's tests/test_replay.py:20-33), and a sample equals the oracle."""
    from elara_b200 import synth
    from elara_b200.gpu_ops import replay_rows, init_rows, ScalarTable
    from elara_b200.ops import gpu_adam
    n, D, K = 262_144, 64, 3
    c = synth.replay_case(n, 4_000_000, D, K, 50, 1234)
    t = {k: torch.from_numpy(v).to(dev) for k, v in c.items()}
    table = ScalarTable(*HYP, 50, dev)
    rp = replay_rows(t['rows'], t['logs'], t['offs'], t['steps'], t['cnt'], D, K, 1234, 0.01, table)
    eg = init_rows(t['rows'], D, 1234, 0.01)
    for s in range(1, 51):
        for k in range(K):
            idx = ((t['cnt'] > k) & (t['steps'][:, k] == s)).nonzero().flatten()
            if idx.numel():
                gpu_adam(eg, idx, t['logs'][t['offs'][idx] + k].contiguous(), *HYP, s)
    assert torch.equal(rp, eg)
    sel = np.arange(0, n, 97)
    sub = {k: c[k][sel] for k in ('rows', 'cnt', 'steps')}
    lg = np.concatenate([c['logs'][c['offs'][i]:c['offs'][i] + c['cnt'][i]] for i in sel])
    so = np.cumsum(sub['cnt'], dtype=np.int64) - sub['cnt']
    want = oracle.replay_rows(sub['rows'], lg, so, sub['steps'], sub['cnt'], D, K, 1234, 0.01, oracle.scalar_table(*HYP, 50))
    assert np.array_equal(bits(rp.cpu().numpy()[sel]), bits(want))
