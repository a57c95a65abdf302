"""Fused assemble (srm2_assemble_f32) against the CPU oracle's init / replay and plain copies: W, fullN and fullL bit for
bit; every group may be empty; shapes the fused kernel does not take fall back to the separate kernels."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)
bits = lambda a: np.ascontiguousarray(a).view(np.uint32)


@pytest.fixture(scope='module')
def dev():
    assert torch.cuda.is_available(), 'these tests need a CUDA device'
    from elara_b200 import _lib
    _lib.lib()
    return torch.device('cuda:0')


def make_case(rng, n, D, K, frac, C=5000, R=4_000_000):
    """Unique rows 0..n-1 of a step, split at random into the five sources (fractions `frac`)."""
    from elara_b200 import synth
    cls = rng.choice(5, size=n, p=frac)
    pos = [np.flatnonzero(cls == c).astype(np.int64) for c in range(5)]
    nh, nN, nL, nF, nS = (len(p) for p in pos)
    c = dict(pos=pos, pool=rng.standard_normal((C, 3, D)).astype(np.float32),
             hit_slot=rng.choice(C, size=nh, replace=False).astype(np.int64),
             N_row=np.concatenate([rng.choice(R, size=max(nN - 1, 0), replace=False), [2**33 + 7]])[:nN].astype(np.int64),
             ff=rng.standard_normal((nF, 3, D)).astype(np.float32), sw=rng.standard_normal((nS, D)).astype(np.float32))
    rc = synth.replay_case(max(nL, 1), R, D, max(K, 1), 50, int(rng.integers(1 << 30)), min_cnt=0)
    for k in ('rows', 'cnt', 'steps', 'offs'):
        rc[k] = rc[k][:nL]
    if K == 0:
        rc['cnt'][:] = 0; rc['steps'] = np.zeros((nL, 0), np.int32); rc['logs'] = np.zeros((0, D), np.float32); rc['offs'][:] = 0
    c['L'] = rc
    return c


@pytest.mark.parametrize('n,D,K,frac', [(6000, 128, 3, (.5, .2, .2, .05, .05)), (3000, 64, 3, (.2, .2, .2, .2, .2)), (500, 16, 1, (1, 0, 0, 0, 0)),
                                        (700, 32, 5, (0, .5, .5, 0, 0)), (400, 64, 0, (.3, .3, .4, 0, 0)), (300, 24, 2, (.2, .2, .2, .2, .2)),
                                        (200, 6, 3, (.2, .2, .2, .2, .2)), (100, 64, 9, (.2, .2, .2, .2, .2))])
def test_assemble_vs_oracle(dev, oracle, n, D, K, frac):
    from elara_b200.gpu_ops import assemble, ScalarTable
    rng = np.random.default_rng(n + D + K)
    c = make_case(rng, n, D, K, frac)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    L = c['L']
    table = ScalarTable(*HYP, 50, dev)
    args = (n, D, t(c['pool']), t(c['pos'][0]), t(c['hit_slot']), t(c['pos'][1]), t(c['N_row']), t(c['pos'][2]), t(L['rows']),
            t(L['logs']), t(L['offs']), t(L['steps']), t(L['cnt']), K, 1234, 0.01, table, t(c['ff']), t(c['pos'][3]), t(c['sw']), t(c['pos'][4]))
    odd = bool(D % 4) or K > 8
    if odd:            # not a shape of the fused kernel: refused unless the caller asks for the separate calls
        with pytest.raises(RuntimeError):
            assemble(*args)
    W, fullN, fullL = assemble(*args, allow_separate_calls=odd)
    want = np.zeros((n, D), np.float32)
    want[c['pos'][0]] = c['pool'][c['hit_slot'], 0]
    if len(c['N_row']):
        wN = oracle.init_rows(c['N_row'], D, 1234, 0.01)
        want[c['pos'][1]] = wN[:, 0]
        assert np.array_equal(bits(fullN.cpu().numpy()), bits(wN))
    else:
        assert fullN is None
    if len(L['rows']):
        wL = oracle.replay_rows(L['rows'], L['logs'], L['offs'], L['steps'], L['cnt'], D, K, 1234, 0.01, oracle.scalar_table(*HYP, 50))
        want[c['pos'][2]] = wL[:, 0]
        assert np.array_equal(bits(fullL.cpu().numpy()), bits(wL))
    else:
        assert fullL is None
    want[c['pos'][3]] = c['ff'][:, 0]
    want[c['pos'][4]] = c['sw']
    assert np.array_equal(bits(W.cpu().numpy()), bits(want))       # the five groups cover every row of W


def test_assemble_skips_bad_positions(dev):
    """A position outside W is not written (and nothing else is): the kernel checks instead of faulting."""
    from elara_b200.gpu_ops import assemble, ScalarTable
    D, n = 64, 10
    e64 = torch.empty(0, dtype=torch.int64, device=dev); e32 = torch.empty(0, dtype=torch.int32, device=dev); ef = torch.empty(0, device=dev)
    sw = torch.arange(3 * D, dtype=torch.float32, device=dev).view(3, D)
    pool = torch.zeros(4, 3, D, device=dev)
    W, _, _ = assemble(n, D, pool, e64, e64, e64, e64, e64, e64, ef, e64, e32, e32, 3, 1, 0.01, ScalarTable(*HYP, 5, dev), ef, e64, sw,
                       torch.tensor([2, -1, n], device=dev))
    torch.cuda.synchronize()
    assert torch.equal(W[2], sw[0])


def test_forward_gather_behind_assemble(dev):
    """emb[p] = W[inv[p]] as the second launch of the assemble call equals torch.index_select (srm2/train.py:427)."""
    from elara_b200.gpu_ops import assemble, gather_rows, ScalarTable
    n, D, nl = 5000, 128, 60_000
    g = torch.Generator(device=dev).manual_seed(3)
    pool = torch.randn(8000, 3, D, device=dev, generator=g)
    hit_slot = torch.randperm(8000, device=dev, generator=g)[:n]
    pos = torch.arange(n, device=dev)
    inv = torch.randint(0, n, (nl,), device=dev, generator=g)
    e64 = torch.empty(0, dtype=torch.int64, device=dev); e32 = torch.empty(0, dtype=torch.int32, device=dev); ef = torch.empty(0, device=dev)
    W, _, _, emb = assemble(n, D, pool, pos, hit_slot, e64, e64, e64, e64, ef, e64, e32, e32, 3, 1, 0.01, ScalarTable(*HYP, 5, dev), ef, e64, ef, e64,
                            inv=inv)
    assert torch.equal(W, pool[hit_slot, 0])
    assert torch.equal(emb, torch.index_select(W, 0, inv))
    assert torch.equal(gather_rows(W, torch.tensor([0, -1, n, 7], device=dev)), torch.stack([W[0], torch.zeros(D, device=dev), torch.zeros(D, device=dev), W[7]]))
