"""The dedup entry point that brings its own scratch (for hosts that are not allowed to allocate device memory where
they call it) against the regular entry point, through the C ABI.

Two calls in a row with different inputs: the built-in scratch area is shared by all calls and still holds the first
call's bitmap when the second starts, so the second result is only right if the entry point clears what it must.
This file sorts last on purpose: a failure here cannot hide the other tests behind `-x`.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(L, ids, n_rows, dev):
    from elara_b200 import _lib
    n = ids.numel()
    cap = min(n, n_rows)
    u = torch.full((cap,), -7, dtype=torch.int64, device=dev); inv = torch.full((n,), -7, dtype=torch.int64, device=dev)
    cnt = torch.full((2,), -7, dtype=torch.int64, device=dev)
    scr = torch.empty(L.srm2_unique_scratch_bytes(n_rows), dtype=torch.uint8, device=dev)
    _lib.check(L.srm2_unique_inverse_i64(ids.data_ptr(), n, n_rows, u.data_ptr(), cap, inv.data_ptr(), cnt.data_ptr(), scr.data_ptr(),
                                         scr.numel(), torch.cuda.current_stream(dev).cuda_stream), 'regular dedup')
    return u, inv, cnt


def _builtin_scratch(L, ids, n_rows, dev):
    from elara_b200 import _lib
    n = ids.numel()
    cap = min(n, n_rows)
    u = torch.full((cap,), -7, dtype=torch.int64, device=dev); inv = torch.full((n,), -7, dtype=torch.int64, device=dev)
    cnt = torch.full((2,), -7, dtype=torch.int64, device=dev)
    _lib.check(L.srm2_unique_inverse_noalloc_i64(ids.data_ptr(), n, n_rows, u.data_ptr(), cap, inv.data_ptr(), cnt.data_ptr(),
                                                 torch.cuda.current_stream(dev).cuda_stream), 'dedup on the built-in scratch')
    return u, inv, cnt


def test_builtin_scratch_dedup_matches_regular_entry_point_twice():
    from elara_b200 import _lib
    assert torch.cuda.is_available()
    dev = torch.device('cuda:0')
    L = _lib.lib()
    max_rows = L.srm2_unique_noalloc_max_rows()
    assert max_rows == 4_194_304
    rng = np.random.default_rng(123)
    # call 1: the largest universe allowed, many distinct ids; call 2: a smaller universe and other ids, so that stale
    # bits of call 1 would show up as extra "unique" rows if the area were not cleared
    cases = [(max_rows, 200_000), (1_000_003, 50_000)]
    for n_rows, n in cases:
        ids_np = np.minimum((rng.pareto(1.1, n) * 40).astype(np.int64), n_rows - 1)
        mask = rng.random(n) < 0.4
        ids_np[mask] = rng.integers(0, n_rows, int(mask.sum()))
        ids_np[:2] = [0, n_rows - 1]
        ids = torch.from_numpy(ids_np).to(dev)
        u0, inv0, c0 = _regular(L, ids, n_rows, dev)
        u1, inv1, c1 = _builtin_scratch(L, ids, n_rows, dev)
        torch.cuda.synchronize(dev)
        nu = int(c0[0])
        assert torch.equal(c0, c1) and int(c1[1]) == 0
        assert torch.equal(u0[:nu], u1[:nu]) and torch.equal(inv0, inv1)          # integer results: exact equality
        ur, invr = np.unique(ids_np, return_inverse=True)
        assert nu == len(ur) and np.array_equal(u1[:nu].cpu().numpy(), ur) and np.array_equal(inv1.cpu().numpy(), invr.reshape(-1))


def test_builtin_scratch_dedup_rejects_universe_beyond_its_limit():
    from elara_b200 import _lib
    dev = torch.device('cuda:0')
    L = _lib.lib()
    ids = torch.tensor([1, 2, 3], dtype=torch.int64, device=dev)
    u = torch.empty(3, dtype=torch.int64, device=dev); inv = torch.empty(3, dtype=torch.int64, device=dev)
    cnt = torch.full((2,), -7, dtype=torch.int64, device=dev)
    rc = L.srm2_unique_inverse_noalloc_i64(ids.data_ptr(), 3, L.srm2_unique_noalloc_max_rows() + 1, u.data_ptr(), 3, inv.data_ptr(),
                                           cnt.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -5 and b'built-in scratch' in L.srm2_status_string(rc)
    torch.cuda.synchronize(dev)
    assert cnt.tolist() == [-7, -7]                                               # nothing was enqueued
    with pytest.raises(RuntimeError, match='built-in scratch'):
        _lib.check(rc, 'dedup on the built-in scratch')
