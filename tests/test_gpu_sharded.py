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


@pytest.mark.parametrize('n,D,W', [(3000, 16, 2), (40000, 128, 4), (90000, 64, 3), (212992, 128, 8)])
def test_pull_exchange_emulated_on_one_gpu(oracle, n, D, W):
    """Pull form of the exchange with all W ranks' buffers on one device (kernels run one after another, nothing waits):
    plan / publish / dispatch_ids for every rank, then every owner's dedup + srm2_reduce_adam_pull_f32 reading the
    gradient rows where the ranks left them.  The W shards must equal the single-process oracle bit for bit."""
    import ctypes as C
    from elara_b200 import _lib, ops
    from elara_b200.gpu_ops import init_rows
    from elara_b200.sharded import local_rows
    dev = torch.device('cuda:0')
    L = _lib.lib()
    R = 50_000
    rng = np.random.default_rng(n + W)
    p = np.arange(1, R + 1, dtype=np.float64) ** -1.1
    perm0 = rng.permutation(R)
    ids = [perm0[rng.choice(R, size=n, p=p / p.sum())].astype(np.int64) for _ in range(W)]
    grads = [(rng.standard_normal((n, D)) * 10.0 ** rng.integers(-3, 4, size=(n, 1))).astype(np.float32) for _ in range(W)]
    t_ids = [torch.from_numpy(x).to(dev) for x in ids]
    t_grads = [torch.from_numpy(x).to(dev) for x in grads]
    cap = 3 * n + 4096                      # the owner of the hottest rows receives well above the average
    st = torch.cuda.current_stream(dev).cuda_stream
    arr = lambda ts: (C.c_void_p * W)(*[t.data_ptr() for t in ts])
    rlid = [torch.full((cap,), -1, dtype=torch.int64, device=dev) for _ in range(W)]
    rsrc = [torch.zeros(cap, dtype=torch.int32, device=dev) for _ in range(W)]
    cmat = [torch.zeros(W * W, dtype=torch.int64, device=dev) for _ in range(W)]
    n_recv = torch.zeros(W, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    nb = L.srm2_route_scratch_bytes(n, W)
    scr = [torch.empty(nb, dtype=torch.uint8, device=dev) for _ in range(W)]
    counts = torch.zeros(W, dtype=torch.int64, device=dev)
    for r in range(W):
        _lib.check(L.srm2_route_plan(t_ids[r].data_ptr(), n, W, counts.data_ptr(), scr[r].data_ptr(), nb, st), 'plan')
        _lib.check(L.srm2_route_publish(counts.data_ptr(), arr(cmat), r, W, st), 'publish')
    for r in range(W):
        _lib.check(L.srm2_route_dispatch_ids(t_ids[r].data_ptr(), n, W, r, cmat[r].data_ptr(), arr(rlid), arr(rsrc), cap,
                                             n_recv[r:].data_ptr(), err.data_ptr(), 0, 0, 0, scr[r].data_ptr(), nb, st), 'dispatch_ids')
    assert int(err.item()) == 0
    # single-process expectation
    all_ids = np.concatenate(ids); all_grads = np.concatenate(grads)
    state = oracle.init_rows(np.arange(R), D, 7, 0.01)
    u, inv = oracle.unique_inverse(all_ids)
    oracle.adam_rows(state, u, oracle.segment_reduce(all_grads, inv, len(u), chunk=oracle.SEGMENT_CHUNK), *HYP, 3)
    sc = ops._scalars(*HYP, 3)
    for d in range(W):
        nl = local_rows(R, W, d)
        assert int(n_recv[d]) == sum(int((x % W == d).sum()) for x in ids)
        pool = init_rows(torch.arange(nl, device=dev) * W + d, D, 7, 0.01)
        uq = torch.empty(min(cap, nl), dtype=torch.int64, device=dev); iv = torch.empty(cap, dtype=torch.int64, device=dev)
        cnt = torch.zeros(2, dtype=torch.int64, device=dev)
        su = torch.empty(L.srm2_unique_scratch_bytes(nl), dtype=torch.uint8, device=dev)
        ss = torch.empty(L.srm2_segment_scratch_bytes(cap, uq.numel(), D), dtype=torch.uint8, device=dev)
        _lib.check(L.srm2_unique_inverse_nd_i64(rlid[d].data_ptr(), cap, n_recv[d:].data_ptr(), nl, uq.data_ptr(), uq.numel(), iv.data_ptr(),
                                                cnt.data_ptr(), su.data_ptr(), su.numel(), st), 'unique')
        _lib.check(L.srm2_reduce_adam_pull_f32(pool.data_ptr(), uq.data_ptr(), arr(t_grads), W, rsrc[d].data_ptr(), iv.data_ptr(), cap,
                                               n_recv[d:].data_ptr(), D, -1, cnt.data_ptr(), uq.numel(), sc, ss.data_ptr(), ss.numel(), st),
                   'reduce_adam_pull')
        assert np.array_equal(pool.cpu().numpy().view(np.uint32), state[d::W].view(np.uint32)), d


@pytest.mark.parametrize('n,D,W,pcap,one_owner', [(3000, 16, 2, 3001, False), (40000, 128, 4, 20000, False), (90000, 64, 3, 40, False),
                                                  (212992, 128, 8, 53248, False), (50000, 24, 2, 30001, False), (6000, 32, 3, 6001, True)])
def test_pull_exchange_with_sums_prepared_at_the_source(oracle, n, D, W, pcap, one_owner):
    """The pull exchange in which the leading lookups of a run that come from one rank are added up by that rank and read
    by the owner as one row (srm2_presum_request / srm2_presum_rows_f32 / srm2_reduce_adam_apply_pull_f32), all W ranks'
    buffers on one device, no barriers (the calls are made in the order the barriers would enforce).  The shards must
    equal the single-process oracle bit for bit — also where the request regions are far too small (pcap = 40: most runs
    stay as they were) — and the requests must cover a good part of the lookups."""
    import ctypes as C
    from elara_b200 import _lib, ops
    from elara_b200.gpu_ops import init_rows
    from elara_b200.sharded import local_rows
    dev = torch.device('cuda:0')
    L = _lib.lib()
    R = 50_000
    rng = np.random.default_rng(n + W)
    p = np.arange(1, R + 1, dtype=np.float64) ** -1.1
    perm0 = rng.permutation(R)
    ids = [perm0[rng.choice(R, size=n, p=p / p.sum())].astype(np.int64) for _ in range(W)]
    if one_owner:                            # every row belongs to rank 1: the other owners receive nothing and ask for nothing
        ids = [x // W * W + 1 for x in ids]
    grads = [(rng.standard_normal((n, D)) * 10.0 ** rng.integers(-3, 4, size=(n, 1))).astype(np.float32) for _ in range(W)]
    for g in grads:
        g[rng.integers(0, n, 50)] = -0.0                         # signed zeros must come out as the one-by-one sum leaves them
    t_ids = [torch.from_numpy(x).to(dev) for x in ids]
    t_grads = [torch.from_numpy(x).to(dev) for x in grads]
    cap = 3 * n + 4096
    st = torch.cuda.current_stream(dev).cuda_stream
    arr = lambda ts: (C.c_void_p * W)(*[t.data_ptr() for t in ts])
    rlid = [torch.full((cap,), -1, dtype=torch.int64, device=dev) for _ in range(W)]
    rsrc = [torch.zeros(cap, dtype=torch.int32, device=dev) for _ in range(W)]
    cmat = [torch.zeros(W * W, dtype=torch.int64, device=dev) for _ in range(W)]
    n_recv = torch.zeros(W, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    nb = L.srm2_route_scratch_bytes(n, W)
    scr = [torch.empty(nb, dtype=torch.uint8, device=dev) for _ in range(W)]
    counts = torch.zeros(W, dtype=torch.int64, device=dev)
    for r in range(W):
        _lib.check(L.srm2_route_plan(t_ids[r].data_ptr(), n, W, counts.data_ptr(), scr[r].data_ptr(), nb, st), 'plan')
        _lib.check(L.srm2_route_publish(counts.data_ptr(), arr(cmat), r, W, st), 'publish')
    for r in range(W):
        _lib.check(L.srm2_route_dispatch_ids(t_ids[r].data_ptr(), n, W, r, cmat[r].data_ptr(), arr(rlid), arr(rsrc), cap,
                                             n_recv[r:].data_ptr(), err.data_ptr(), 0, 0, 0, scr[r].data_ptr(), nb, st), 'dispatch_ids')
    assert int(err.item()) == 0
    all_ids = np.concatenate(ids); all_grads = np.concatenate(grads)
    state = oracle.init_rows(np.arange(R), D, 7, 0.01)
    u, inv = oracle.unique_inverse(all_ids)
    oracle.adam_rows(state, u, oracle.segment_reduce(all_grads, inv, len(u), chunk=oracle.SEGMENT_CHUNK), *HYP, 3)
    sc = ops._scalars(*HYP, 3)
    # per rank: request buffer [W][pcap][12], counts [W], buffer of sums [W][pcap][D]
    req = [torch.zeros(W * pcap * 12, dtype=torch.int32, device=dev) for _ in range(W)]
    req_n = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(W)]
    outbox = [torch.full((W * pcap * D,), float('nan'), device=dev) for _ in range(W)]
    req_count = torch.zeros(32, dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)

    keep = []

    def presum(rank):
        ps = _lib.Presum()
        ps.world, ps.rank, ps.cap, ps.timeout_ns, ps.err, ps.ticket = W, rank, pcap, 10**9, err.data_ptr(), 0
        ps.peer_req, ps.peer_req_n = C.cast(arr(req), C.c_void_p), C.cast(arr(req_n), C.c_void_p)
        ps.req_count, ps.req, ps.req_n = req_count.data_ptr(), req[rank].data_ptr(), req_n[rank].data_ptr()
        # where rank `rank` stores what owner o asked for: region `rank` of o's buffer of sums
        keep.append((C.c_void_p * W)(*[outbox[o][rank * pcap * D:].data_ptr() for o in range(W)]))
        ps.peer_out, ps.done = C.cast(keep[-1], C.c_void_p), done.data_ptr()
        return ps

    owners = []
    for d in range(W):                       # every owner: dedup, index half, requests
        nl = local_rows(R, W, d)
        pool = init_rows(torch.arange(nl, device=dev) * W + d, D, 7, 0.01)
        uq = torch.empty(min(cap, nl), dtype=torch.int64, device=dev); iv = torch.empty(cap, dtype=torch.int64, device=dev)
        cnt = torch.zeros(2, dtype=torch.int64, device=dev)
        su = torch.empty(L.srm2_unique_scratch_bytes(nl), dtype=torch.uint8, device=dev)
        ss = torch.empty(L.srm2_segment_scratch_bytes(cap, uq.numel(), D), dtype=torch.uint8, device=dev)
        _lib.check(L.srm2_unique_inverse_nd_i64(rlid[d].data_ptr(), cap, n_recv[d:].data_ptr(), nl, uq.data_ptr(), uq.numel(), iv.data_ptr(),
                                                cnt.data_ptr(), su.data_ptr(), su.numel(), st), 'unique')
        _lib.check(L.srm2_reduce_adam_index(uq.data_ptr(), rsrc[d].data_ptr(), iv.data_ptr(), cap, n_recv[d:].data_ptr(), D, -1, cnt.data_ptr(),
                                            uq.numel(), 0, ss.data_ptr(), ss.numel(), st), 'index')
        ps = presum(d)
        _lib.check(L.srm2_presum_request(cap, n_recv[d:].data_ptr(), D, uq.numel(), ss.data_ptr(), ss.numel(), C.byref(ps), st), 'request')
        owners.append((pool, uq, cnt, ss))
    for r in range(W):                       # every source: the sums its peers asked for
        ps = presum(r)
        _lib.check(L.srm2_presum_rows_f32(t_grads[r].data_ptr(), n, D, C.byref(ps), st), 'presum_rows')
    assert int(err.item()) == 0
    asked = torch.stack(req_n).cpu().numpy()[:, :W]
    assert asked.max() <= pcap and all(asked[r, r] == 0 for r in range(W))
    if pcap > 1000:                          # every row that left its rank is part of a request; far fewer requests than rows
        taken = sum(int(req[r].view(W, pcap, 12)[o, :asked[r, o], 0].sum()) for r in range(W) for o in range(W))
        assert taken == sum(int((x % W != r).sum()) for r, x in enumerate(ids))
        assert asked.sum() < 0.7 * taken
    else:
        assert asked.sum() == pcap * W * (W - 1)              # every region full
    for d in range(W):                       # every owner: run sums + Adam
        pool, uq, cnt, ss = owners[d]
        p_out = (C.c_void_p * W)(*[outbox[d][s_ * pcap * D:].data_ptr() for s_ in range(W)])     # region s of the owner's own buffer
        _lib.check(L.srm2_reduce_adam_apply_pull_f32(pool.data_ptr(), uq.data_ptr(), arr(t_grads), p_out, err.data_ptr(), W, cap,
                                                     n_recv[d:].data_ptr(), D, -1, cnt.data_ptr(), uq.numel(), sc, ss.data_ptr(), ss.numel(), st),
                   'apply_pull')
        assert np.array_equal(pool.cpu().numpy().view(np.uint32), state[d::W].view(np.uint32)), d
    # a set status word: the update kernels leave the shard as it is
    pool, uq, cnt, ss = owners[0]
    before = pool.clone()
    err.fill_(2)
    p_out = (C.c_void_p * W)(*[outbox[0][s_ * pcap * D:].data_ptr() for s_ in range(W)])
    _lib.check(L.srm2_reduce_adam_apply_pull_f32(pool.data_ptr(), uq.data_ptr(), arr(t_grads), p_out, err.data_ptr(), W, cap, n_recv.data_ptr(), D, -1,
                                                 cnt.data_ptr(), uq.numel(), sc, ss.data_ptr(), ss.numel(), st), 'apply_pull')
    assert torch.equal(pool.view(torch.int32), before.view(torch.int32))


def test_engine_world1_pipelined_equals_step_by_step(oracle):
    """run_steps at world size 1 (index half of step s+1 on a side stream while the sum half of step s runs) against
    step() on a second engine and against the oracle."""
    from elara_b200 import synth
    from elara_b200.sharded import ShardedSparseAdam
    dev = torch.device('cuda:0')
    R, D, batch = 300_000, 128, 1024
    sizes, offs = synth.table_sizes(R, 26, lo=4, hi=100_000, seed=5)
    mk = lambda: ShardedSparseAdam(R, D, 1, 0, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26)
    eng, ref = mk(), mk()
    st = oracle.init_rows(np.arange(R), D, 42, 0.01)
    batches = []
    for step in range(1, 8):
        ids = synth.zipf_lookups(sizes, offs, batch, 1.1, 11, step)
        grad = synth.normal_f32((len(ids), D), 1e-3, 11, step)
        batches.append((torch.from_numpy(ids).to(dev), torch.from_numpy(grad).to(dev)))
        u, inv = oracle.unique_inverse(ids)
        oracle.adam_rows(st, u, oracle.segment_reduce(grad, inv, len(u)), *HYP, step)
        ref.step(*batches[-1], step)
    counts = eng.run_steps(batches[:4], 1) + eng.run_steps(batches[4:], 5)
    eng2 = mk(); eng2.host_loop = True                       # the same stages issued from Python instead of srm2_staged_steps
    counts2 = eng2.run_steps(batches[:1], 1) + eng2.run_steps(batches[1:], 2)
    torch.cuda.synchronize()
    assert [int(c[0]) for c in counts] == [len(np.unique(i.cpu().numpy())) for i, _ in batches]
    assert [int(c[0]) for c in counts2] == [int(c[0]) for c in counts]
    assert torch.equal(eng.pool.view(torch.int32), ref.pool.view(torch.int32))
    assert torch.equal(eng2.pool.view(torch.int32), ref.pool.view(torch.int32))
    assert np.array_equal(eng.pool.cpu().numpy().view(np.uint32), st.view(np.uint32))


def test_peer_barrier_wait_is_bounded():
    """The barrier kernel of the exchange gives up after its time limit and reports it: here `rank 1` never arrives (its
    ticket array is a buffer that nothing writes), so rank 0 flags status 2 after 2 ms and the context stays usable; a
    second barrier whose tickets are already there passes without a flag."""
    import ctypes as C
    from elara_b200 import _lib
    dev = torch.device('cuda:0')
    L = _lib.lib()
    mine = torch.zeros(16, dtype=torch.int64, device=dev)
    other = torch.zeros(16, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    arr = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    st = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(L.srm2_peer_barrier(arr, 0, 2, 1, err.data_ptr(), 2_000_000, 0, st), 'barrier')
    torch.cuda.synchronize()
    assert int(err.item()) == 2
    assert int(other[0]) == 1 and int(mine[0]) == 1            # its own tickets were delivered
    err.zero_(); mine[1] = 2                                    # "rank 1" has arrived at barrier 2
    _lib.check(L.srm2_peer_barrier(arr, 0, 2, 2, err.data_ptr(), 2_000_000, 0, st), 'barrier')
    torch.cuda.synchronize()
    assert int(err.item()) == 0


def test_failed_exchange_leaves_the_shard_untouched():
    """Containment: a barrier that runs out (the peer never arrives) zeroes the step's count of received lookups, and the
    flag is sticky, so the update kernels of that step and of the next one see an empty batch: no row of the shard changes
    although the receive buffer holds (stale) lookups.  A healthy barrier leaves the count alone and the update runs."""
    import ctypes as C
    from elara_b200 import _lib, ops
    from elara_b200.gpu_ops import init_rows
    dev = torch.device('cuda:0')
    L = _lib.lib()
    R, D, n = 20_000, 64, 5_000
    pool = init_rows(torch.arange(R, device=dev), D, 3, 0.01)
    before = pool.clone()
    ids = torch.randint(0, R, (n,), device=dev)
    grad = torch.randn(n, D, device=dev) * 1e-3
    mine = torch.zeros(16, dtype=torch.int64, device=dev)
    other = torch.zeros(16, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    arr = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    st = torch.cuda.current_stream(dev).cuda_stream

    def update(n_recv, step):
        u, inv, count = ops.unique_inverse(ids, R, sync=False, n_dev=n_recv)
        ops.reduce_adam(pool, u, grad, inv, *HYP, step, count=count, order=ops.ORDER_RUNS, n_dev=n_recv)
        return int(count[0])
    n_recv = torch.full((1,), n, dtype=torch.int64, device=dev)
    _lib.check(L.srm2_peer_barrier(arr, 0, 2, 1, err.data_ptr(), 2_000_000, n_recv.data_ptr(), st), 'barrier')     # rank 1 never arrives
    assert update(n_recv, 1) == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 2 and int(n_recv.item()) == 0
    assert torch.equal(pool.view(torch.int32), before.view(torch.int32))
    n_recv.fill_(n); mine[1] = 2                                 # the peer is there for barrier 2, but the failure is sticky
    _lib.check(L.srm2_peer_barrier(arr, 0, 2, 2, err.data_ptr(), 2_000_000, n_recv.data_ptr(), st), 'barrier')
    assert update(n_recv, 1) == 0
    assert torch.equal(pool.view(torch.int32), before.view(torch.int32))
    err.zero_(); n_recv.fill_(n); mine[1] = 3                    # cleared by the host: a healthy barrier changes nothing
    _lib.check(L.srm2_peer_barrier(arr, 0, 2, 3, err.data_ptr(), 2_000_000, n_recv.data_ptr(), st), 'barrier')
    assert update(n_recv, 1) == len(torch.unique(ids))
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and int(n_recv.item()) == n
    assert not torch.equal(pool.view(torch.int32), before.view(torch.int32))
