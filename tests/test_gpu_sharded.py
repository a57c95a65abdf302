"""Device side of the row-sharded step on one GPU: owner routing against a NumPy stable partition, and the sharded
engine at world size 1 against the oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)


@pytest.mark.parametrize('n,D,world', [(1, 4, 2), (5000, 16, 2), (70000, 128, 8), (212992, 128, 8), (9000, 24, 3), (4097, 8, 1)])
def test_route_by_owner(n, D, world):
    from elara_b200.sharded import ShardedSparseAdam
    dev = torch.device('cuda:0')
    rng = np.random.default_rng(n + world)
    ids = np.minimum((rng.pareto(1.1, n) * 50).astype(np.int64), 10**6 - 1)
    grad = rng.standard_normal((n, D)).astype(np.float32)
    eng = ShardedSparseAdam.__new__(ShardedSparseAdam)
    eng.world, eng.D, eng.dev = world, D, dev
    eng._lid = torch.empty(n, dtype=torch.int64, device=dev); eng._grad = torch.empty(n, D, device=dev)
    eng._counts = torch.empty(world, dtype=torch.int64, device=dev)
    lids, g, counts = eng.route(torch.from_numpy(ids).to(dev), torch.from_numpy(grad).to(dev))
    perm = np.argsort(ids % world, kind='stable')
    assert np.array_equal(counts.cpu().numpy(), np.bincount(ids % world, minlength=world))
    assert np.array_equal(lids.cpu().numpy(), ids[perm] // world)
    assert np.array_equal(g.cpu().numpy().view(np.uint32), grad[perm].view(np.uint32))


def test_engine_world1_vs_oracle(oracle):
    from elara_b200 import synth
    from elara_b200.sharded import ShardedSparseAdam
    dev = torch.device('cuda:0')
    R, D, batch = 300_000, 128, 1024
    sizes, offs = synth.table_sizes(R, 26, lo=4, hi=100_000, seed=5)
    eng = ShardedSparseAdam(R, D, 1, 0, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26)
    st = oracle.init_rows(np.arange(R), D, 42, 0.01)
    for step in range(1, 5):
        ids = synth.zipf_lookups(sizes, offs, batch, 1.1, 9, step)
        grad = synth.normal_f32((len(ids), D), 1e-3, 9, step)
        c = eng.step(torch.from_numpy(ids).to(dev), torch.from_numpy(grad).to(dev), step)
        u, inv = oracle.unique_inverse(ids)
        oracle.adam_rows(st, u, oracle.segment_reduce(grad, inv, len(u)), *HYP, step)
        assert int(c[0]) == len(u) and int(c[1]) == 0
    assert np.array_equal(eng.pool.cpu().numpy().view(np.uint32), st.view(np.uint32))
