"""Dedup, segment-reduce and the fused reduce+Adam kernels against the oracle, against PyTorch's own CUDA operator
run live, and against the known-answer vectors that operator produced (tests/golden/segreduce_cuda.npz)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.fixture(scope='module')
def dev():
    assert torch.cuda.is_available()
    return torch.device('cuda:0')


def order_sensitive(rng, n, D):
    g = (rng.standard_normal((n, D)) * 10.0 ** rng.integers(-3, 4, (n, 1))).astype(np.float32)
    g[rng.random(n) < 0.02] = 0.0
    g[rng.random(n) < 0.02] = -0.0
    return g


# ------------------------------------------------------------------------------------------------ dedup
@pytest.mark.parametrize('n,n_rows', [(1, 1), (1, 5), (1000, 50), (5000, 131072), (5000, 131073), (70000, 131071), (212992, 33_800_000),
                                      (50000, 4_194_304 + 17)])
def test_unique_inverse(dev, oracle, n, n_rows):
    from elara_b200.ops import unique_inverse
    rng = np.random.default_rng(n + n_rows)
    ids = np.minimum((rng.pareto(1.1, n) * 3).astype(np.int64), n_rows - 1)
    mask = rng.random(n) < 0.3
    ids[mask] = rng.integers(0, n_rows, int(mask.sum()))
    ids[:3] = [0, n_rows - 1, min(n_rows - 1, 131071)][:min(3, n)]
    u, inv = unique_inverse(torch.from_numpy(ids).to(dev), n_rows)
    ur, invr = oracle.unique_inverse(ids)
    tu, tinv = torch.unique(torch.from_numpy(ids), return_inverse=True)
    assert np.array_equal(ur, tu.numpy()) and np.array_equal(invr, tinv.numpy())
    assert u.dtype == torch.int64 and inv.dtype == torch.int64
    assert np.array_equal(u.cpu().numpy(), ur) and np.array_equal(inv.cpu().numpy(), invr)


def test_unique_inverse_edges(dev):
    from elara_b200.ops import unique_inverse
    u, inv = unique_inverse(torch.empty(0, dtype=torch.int64, device=dev), 100)
    assert u.numel() == 0 and inv.numel() == 0
    with pytest.raises(RuntimeError):
        unique_inverse(torch.tensor([1, 100], device=dev), 100)
    with pytest.raises(RuntimeError):
        unique_inverse(torch.tensor([-1, 3], device=dev), 100)
    # the call can be repeated on the same scratch, results do not depend on what was there before
    a = torch.tensor([5, 3, 5, 99, 0], device=dev)
    for _ in range(3):
        u, inv = unique_inverse(a, 100)
        assert u.tolist() == [0, 3, 5, 99] and inv.tolist() == [2, 1, 2, 3, 0]


# ---------------------------------------------------------------------------------------- segment-reduce
CASES = [(1, 16, 1), (33, 16, 3), (100, 128, 7), (1000, 4, 40), (3072, 16, 40), (3072, 24, 3), (3073, 16, 900), (3073, 16, 3), (5000, 64, 40),
         (20000, 128, 600), (70000, 16, 5000), (212992, 128, 50000), (9000, 8, 1), (200000, 64, 30), (120000, 128, 9)]


@pytest.mark.parametrize('n,D,nk', CASES)
def test_segment_reduce_vs_oracle(dev, oracle, n, D, nk):
    from elara_b200.ops import segment_reduce
    rng = np.random.default_rng(n * 7 + D)
    p = np.arange(1, nk + 1, dtype=np.float64) ** -1.1
    keys = rng.choice(nk, size=n, p=p / p.sum())
    _, inv = np.unique(keys, return_inverse=True)
    inv = inv.reshape(-1).astype(np.int64); nu = int(inv.max()) + 1
    grad = order_sensitive(rng, n, D)
    out = segment_reduce(torch.from_numpy(grad).to(dev), torch.from_numpy(inv).to(dev), nu)
    want = oracle.segment_reduce(grad, inv, nu)
    assert np.array_equal(bits(out.cpu().numpy()), bits(want))


def test_segment_reduce_rows_without_lookups(dev, oracle):
    from elara_b200.ops import segment_reduce
    rng = np.random.default_rng(9)
    for n in (500, 6000):
        inv = rng.choice([0, 3, 4, 9], size=n).astype(np.int64)
        grad = order_sensitive(rng, n, 16)
        out = segment_reduce(torch.from_numpy(grad).to(dev), torch.from_numpy(inv).to(dev), 12).cpu().numpy()
        assert np.array_equal(bits(out), bits(oracle.segment_reduce(grad, inv, 12)))
        assert not out[[1, 2, 5, 6, 7, 8, 10, 11]].any()


@pytest.mark.parametrize('n,D,nk', [(2000, 16, 50), (3072, 128, 300), (3073, 128, 1500), (20000, 64, 600), (212992, 128, 50000),
                                    (1_703_936, 128, 300000)])
def test_segment_reduce_vs_torch_operator(dev, n, D, nk):
    """Live comparison with the operator the reference calls (srm2/train.py:429), on inputs where that operator is
    run-to-run deterministic (many unique rows, or at most 3072 lookups)."""
    from elara_b200.ops import segment_reduce
    rng = np.random.default_rng(n + D)
    p = np.arange(1, nk + 1, dtype=np.float64) ** -1.1
    keys = rng.choice(nk, size=n, p=p / p.sum())
    _, inv = np.unique(keys, return_inverse=True)
    inv = torch.from_numpy(inv.reshape(-1).astype(np.int64)).to(dev); nu = int(inv.max()) + 1
    grad = torch.from_numpy(order_sensitive(rng, n, D)).to(dev)
    ref = torch.ops.aten.embedding_dense_backward(grad, inv, nu, -1, False)
    ref2 = torch.ops.aten.embedding_dense_backward(grad, inv, nu, -1, False)
    assert torch.equal(ref.view(torch.int32), ref2.view(torch.int32)), 'the torch operator was not deterministic on this input'
    out = segment_reduce(grad, inv, nu)
    assert torch.equal(out.view(torch.int32), ref.view(torch.int32))


def test_segment_reduce_golden(dev, golden_dir):
    from elara_b200.ops import segment_reduce
    f = golden_dir / 'segreduce_cuda.npz'
    g = np.load(f)
    for ci in range(int(g['n_cases'])):
        grad, inv, nu = g[f'c{ci}_grad'], g[f'c{ci}_inv'], int(g[f'c{ci}_nu'])
        out = segment_reduce(torch.from_numpy(grad).to(dev), torch.from_numpy(inv).to(dev), nu)
        assert np.array_equal(bits(out.cpu().numpy()), bits(g[f'c{ci}_out'])), ci


# ------------------------------------------------------------------------------------------- fused + Adam
@pytest.mark.parametrize('n,D,R', [(2500, 16, 4000), (40000, 64, 30000), (212992, 128, 400000)])
def test_reduce_adam_fused_equals_two_calls_and_oracle(dev, oracle, n, D, R):
    from elara_b200.ops import unique_inverse, segment_reduce, reduce_adam, gpu_adam
    from elara_b200.gpu_ops import init_rows
    rng = np.random.default_rng(n)
    ids = np.minimum((rng.pareto(1.1, n) * 5).astype(np.int64), R - 1)
    mask = rng.random(n) < 0.2
    ids[mask] = rng.integers(0, R, int(mask.sum()))
    pool_a = init_rows(torch.arange(R, device=dev), D, 42, 0.01)
    pool_b = pool_a.clone(); pool_c = pool_a.clone()
    st = pool_a.cpu().numpy().copy()
    for step in range(1, 4):
        grad = order_sensitive(rng, n, D) * np.float32(1e-3)
        ids_d = torch.from_numpy(ids).to(dev); grad_d = torch.from_numpy(grad).to(dev)
        # (a) two calls, as the reference driver does
        u, inv = unique_inverse(ids_d, R)
        gW = segment_reduce(grad_d, inv, u.numel())
        gpu_adam(pool_a, u, gW, *HYP, step)
        # (b) fused, host-known count   (c) fused, count stays on the device
        reduce_adam(pool_b, u, grad_d, inv, *HYP, step, n_unique=u.numel())
        ub, invb, count = unique_inverse(ids_d, R, sync=False)
        reduce_adam(pool_c, ub, grad_d, invb, *HYP, step, count=count)
        # oracle
        uo, invo = oracle.unique_inverse(ids)
        oracle.adam_rows(st, uo, oracle.segment_reduce(grad, invo, len(uo)), *HYP, step)
        ids = np.roll(ids, 17)
    assert torch.equal(pool_a.view(torch.int32), pool_b.view(torch.int32))
    assert torch.equal(pool_a.view(torch.int32), pool_c.view(torch.int32))
    assert np.array_equal(bits(pool_a.cpu().numpy()), bits(st))


# ------------------------------------------------------------------------------------------------ large inputs
def _zipf_inverse(rng, n, nu):
    """Inverse indices of n lookups over nu rows with a heavy head (every row named at least once)."""
    inv = np.minimum((rng.pareto(1.05, n) * 40).astype(np.int64), nu - 1)
    mask = rng.random(n) < 0.5
    inv[mask] = rng.integers(0, nu, int(mask.sum()))
    inv[:nu] = rng.permutation(nu)
    return inv


def test_segment_reduce_above_two_million_lookups(dev, oracle):
    """2^21 lookups used to be a limit of the plan's packed scan; there is none now (lookup positions are 32-bit)."""
    from elara_b200.ops import segment_reduce, reduce_adam
    from elara_b200.gpu_ops import init_rows
    rng = np.random.default_rng(21)
    n, nu, D = (1 << 21) + 4097, 300_000, 8
    inv = _zipf_inverse(rng, n, nu)
    g = order_sensitive(rng, n, D)
    got = segment_reduce(torch.from_numpy(g).to(dev), torch.from_numpy(inv).to(dev), nu).cpu().numpy()
    want = oracle.segment_reduce(g, inv, nu)
    assert np.array_equal(bits(got), bits(want))
    pool = init_rows(torch.arange(nu, device=dev), D, 3, 0.01)
    st = oracle.init_rows(np.arange(nu), D, 3, 0.01)
    reduce_adam(pool, torch.arange(nu, device=dev), torch.from_numpy(g).to(dev), torch.from_numpy(inv).to(dev), *HYP, 2, n_unique=nu)
    oracle.adam_rows(st, np.arange(nu), want, *HYP, 2)
    assert np.array_equal(bits(pool.cpu().numpy()), bits(st))


def test_segment_reduce_sort_with_separate_scan(dev, oracle):
    """More than 2^23 (tile, digit) histogram entries: the radix passes scan their histogram with the single-CTA scan kernel
    (in place) instead of deriving the offsets inside the scatter kernel."""
    from elara_b200.ops import segment_reduce
    rng = np.random.default_rng(23)
    n, nu, D = 4_300_000, 4_000_000, 4
    inv = rng.integers(0, nu, n)
    inv[:nu] = rng.permutation(nu)
    inv[nu:nu + 100_000] = 7                       # one long row as well
    g = order_sensitive(rng, n, D)
    got = segment_reduce(torch.from_numpy(g).to(dev), torch.from_numpy(inv).to(dev), nu).cpu().numpy()
    assert np.array_equal(bits(got), bits(oracle.segment_reduce(g, inv, nu)))


def test_segment_reduce_size_limit_is_reported(dev):
    """Lookup positions are 32-bit: a count of 2^31 or more is refused on the host, before anything is enqueued."""
    from elara_b200 import _lib
    L = _lib.lib()
    t = torch.zeros(64, device=dev)
    i = torch.zeros(64, dtype=torch.int64, device=dev)
    scr = torch.zeros(4096, dtype=torch.uint8, device=dev)
    rc = L.srm2_segment_reduce_f32(t.data_ptr(), i.data_ptr(), 1 << 31, 4, 16, 0, 16, 1, t.data_ptr(), scr.data_ptr(), scr.numel(), 0)
    assert rc == _lib.SRM2_ERR_UNSUPPORTED
    with pytest.raises(RuntimeError, match='outside what the kernels are built for|size'):
        _lib.check(rc, 'segment_reduce')
