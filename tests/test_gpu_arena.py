"""Capacity-tier arenas in HBM against the reference's own host copies (cpu_gather / cpu_scatter / cpu_adam of
srm2/csrc/srm2_cpu.cpp:22-81, compiled into oracle/_ref) on the same arenas, ids and payloads: byte for byte."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)


@pytest.fixture(scope='module')
def dev():
    if not torch.cuda.is_available():
        pytest.skip('needs a CUDA device')
    return torch.device('cuda:0')


@pytest.fixture(scope='module')
def E():
    from oracle import oracle as O
    e = O.ref_cpu()
    if e is None:
        pytest.skip('the compiled reference extension is missing (python oracle/build_ref.py --ref <checkout>)')
    return e


def bits(t):
    return t.contiguous().view(torch.int32)


@pytest.mark.parametrize('R,D,n', [(5000, 128, 3000), (20_000, 64, 20_000), (300, 8, 7), (1000, 24, 0)])
def test_arena_ops_equal_the_reference_host_copies(dev, E, R, D, n):
    from elara_b200.arena import HbmArenaStore
    g = torch.Generator().manual_seed(R + D)
    st = HbmArenaStore(R, D, dev)
    h_mat = torch.randn(st.mat_cap + 1, 3, D, generator=g)
    h_mat[:, 2].abs_()                                         # second moments are never negative
    h_log = torch.randn(st.log_cap + 1, 1, D, generator=g)
    st.mat.copy_(h_mat); st.logs.copy_(h_log)
    pick = lambda cap: torch.randperm(cap + 1, generator=g)[:n].contiguous()          # distinct physical ids, trash row included
    # gathers: weights only (1 of 3 components), full records, log entries
    for which, host, ncomp in (('mat', h_mat, 1), ('mat', h_mat, 3), ('log', h_log, 1)):
        ids = pick(host.shape[0] - 1)
        want = torch.empty(n, ncomp, D)
        E.cpu_gather(host, ids, want, ncomp, 4)
        got = st.gather(which, ids.to(dev), ncomp)
        assert torch.equal(bits(got.cpu()), bits(want))
    # scatters: full records and single components into MAT, entries into the log arena
    for which, host, Wc in (('mat', h_mat, 3), ('mat', h_mat, 1), ('log', h_log, 1)):
        ids = pick(host.shape[0] - 1)
        src = torch.randn(n, Wc, D, generator=g)
        E.cpu_scatter(host, ids, src, 4)
        st.scatter(which, ids.to(dev), src.to(dev))
        assert torch.equal(bits(st._arena(which).cpu()), bits(host))
    # Adam on MAT records by physical id (the scattered payloads were arbitrary: make the second moments valid again)
    h_mat[:, 2].abs_(); st.mat[:, 2].abs_()
    ids = pick(st.mat_cap - 1).sort().values
    grad = torch.randn(n, D, generator=g) * 1e-3
    if n:
        E.cpu_adam(h_mat, ids, grad, *HYP, 7, 4)
        st.adam(ids.to(dev), grad.to(dev), *HYP, 7)
    assert torch.equal(bits(st.mat.cpu()), bits(h_mat))
    assert not st.bad_ids_seen()


def test_arena_rejects_ids_outside_the_arena(dev):
    from elara_b200.arena import HbmArenaStore
    st = HbmArenaStore(100, 8, dev)
    st.mat.zero_()
    out = st.gather('mat', torch.tensor([5, 10_000, -3], device=dev), 3)
    torch.cuda.synchronize()
    assert st.bad_ids_seen() and not st.bad_ids_seen()
    assert torch.equal(out[0].cpu(), torch.zeros(3, 8))
    st.scatter('mat', torch.tensor([101, 7], device=dev), torch.ones(2, 3, 8, device=dev))       # 101 > trash row 100
    assert st.bad_ids_seen()
    assert float(st.mat[7].sum()) == 24.0 and float(st.mat.sum()) == 24.0
    with pytest.raises(RuntimeError):
        st.gather('mat', torch.tensor([1], dtype=torch.int32, device=dev), 1)
