"""The library under the reference's own Python, on the GPU.

Needs the reference's package staged beside its compiled extensions in oracle/_ref/ (oracle/build_ref.py does both;
the folder is untracked test infrastructure and travels with the working tree).  Every test here skips when it is absent.

  * GPU against GPU: the reference's Triton gpu_adam / init_rows / replay_rows (srm2/ops.py:42-67, srm2/gpu_ops.py:26-99)
    and this library's kernels on the same inputs, bit for bit, at the shapes of the reference's own tests
    (tests/test_ops.py:11-24, tests/test_replay.py:9-33) and at the stated sizes of the first two benchmark
    configurations (1,000,000 x 16 table, 100 steps of 65,536 rows; replay of 262,144 rows x 64).
  * End to end: the reference's ELARAPlanner(dir_impl='cpp') + ELARAExecutor (srm2/elara.py:107-604) driven twice over the
    same seeded id and gradient stream — stock, and with gpu_adam, init_rows, replay_rows, ScalarTable and dir_ext
    re-pointed at this library — then the 17 directory tensors (without their trash destinations), the planner's
    residency lists, the resident pool, the gradient histories, the materialised arena rows and every live log row are
    compared bit for bit.  First at a middle size, then at the state-directory configuration's own size (33.8 M-row
    store, 8 M-row pool, K = 3, 212,992 lookups per step, 100 steps).
"""
import collections
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / 'oracle' / '_ref'
HYP = (1e-3, 0.9, 0.999, 1e-8)


@pytest.fixture(scope='module')
def dev():
    if not torch.cuda.is_available():
        pytest.skip('needs a CUDA device')
    return torch.device('cuda:0')


@pytest.fixture(scope='module')
def ref(dev):
    """The reference's srm2 package with its two compiled extensions already loaded (no JIT build on the box)."""
    if not (REF / 'srm2' / 'ops.py').exists():
        pytest.skip('oracle/_ref/srm2 is not staged (python oracle/build_ref.py --ref <reference checkout>)')
    from oracle import oracle as O
    E, Dx = O.ref_cpu(), O.ref_dir()
    if E is None or Dx is None:
        pytest.skip('the compiled reference extensions are missing')
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import srm2.ops as rops
    rops._ext, rops._dir = E, Dx               # what ext() / dir_ext() return once loaded (srm2/ops.py:19-39)
    import srm2.gpu_ops as rgpu
    import srm2.elara as relara
    import srm2.executor as rexec
    return dict(ops=rops, gpu_ops=rgpu, elara=relara, executor=rexec, E=E, Dx=Dx)


def same_bits(a, b):
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.int32), b.contiguous().view(torch.int32))


# ------------------------------------------------------------------------------------------------ GPU against GPU
def test_adam_reference_test_shapes(dev, ref):
    """tests/test_ops.py:11-24 with this library as a third party: CPU == reference GPU == this library."""
    from elara_b200.ops import gpu_adam
    g0 = torch.Generator().manual_seed(0)
    R, D = 200_000, 128
    host = torch.randn(R, 3, D, generator=g0) * 0.05
    host[:, 1:] = 0
    theirs, ours = host.clone().to(dev), host.clone().to(dev)
    for step in range(1, 7):
        rows = torch.randperm(R, generator=g0)[:30000].sort().values
        grad = torch.randn(len(rows), D, generator=g0) * (10.0 ** (step % 3 - 2))
        ref['E'].cpu_adam(host, rows, grad, *HYP, step, 16)
        ref['ops'].gpu_adam(theirs, rows.to(dev), grad.to(dev), *HYP, step)
        gpu_adam(ours, rows.to(dev), grad.to(dev), *HYP, step)
    torch.cuda.synchronize()
    assert same_bits(theirs, ours)
    assert same_bits(host, ours.cpu())


def test_adam_one_million_by_16_hundred_steps(dev, ref):
    from elara_b200 import synth
    from elara_b200.ops import gpu_adam
    from elara_b200.gpu_ops import init_rows
    R, D, n = 1_000_000, 16, 65_536
    ours = init_rows(torch.arange(R, device=dev), D, 42, 0.01)
    theirs = ref['gpu_ops'].init_rows(torch.arange(R, device=dev), D, 42, 0.01)
    assert same_bits(ours, theirs)
    gen = torch.Generator(device=dev).manual_seed(7)
    for step in range(1, 101):
        rows = torch.from_numpy(synth.zipf_rows_without_replacement(R, n, 1.05, 42, step)).to(dev)
        grad = torch.randn(n, D, device=dev, generator=gen) * 1e-3
        gpu_adam(ours, rows, grad, *HYP, step)
        ref['ops'].gpu_adam(theirs, rows, grad, *HYP, step)
    torch.cuda.synchronize()
    assert same_bits(ours, theirs)


def test_init_and_replay_reference_test_shapes(dev, ref):
    """tests/test_replay.py:9-33: gaps between the rows' log slices (offs = i*K), cnt 0..3, steps up to 1200."""
    from elara_b200.gpu_ops import init_rows, replay_rows, ScalarTable
    D, K, seed, bound = 128, 3, 1234, 0.01
    g0 = torch.Generator().manual_seed(5)
    rows = torch.randint(0, 30_000_000, (5000,), dtype=torch.int64, generator=g0).unique().to(dev)
    n = rows.numel()
    st = torch.stack([torch.randint(1, 400, (n,), generator=g0), torch.randint(400, 800, (n,), generator=g0),
                      torch.randint(800, 1200, (n,), generator=g0)], 1).to(torch.int32).to(dev)
    g = (torch.randn(n, K, D, generator=g0) * 1e-2).to(dev)
    cnt = torch.randint(0, K + 1, (n,), dtype=torch.int32, generator=g0).to(dev)
    offs = torch.arange(n, device=dev) * K
    t_ref = ref['gpu_ops'].ScalarTable(*HYP, 1300, dev)
    t_our = ScalarTable(*HYP, 1300, dev)
    assert same_bits(t_ref.t, t_our.t)
    assert same_bits(ref['gpu_ops'].init_rows(rows, D, seed, bound), init_rows(rows, D, seed, bound))
    a = ref['gpu_ops'].replay_rows(rows, g.reshape(-1, D).contiguous(), offs, st.contiguous(), cnt, D, K, seed, bound, t_ref)
    b = replay_rows(rows, g.reshape(-1, D).contiguous(), offs, st.contiguous(), cnt, D, K, seed, bound, t_our)
    torch.cuda.synchronize()
    assert same_bits(a, b)


def test_replay_262144_rows_by_64(dev, ref):
    from elara_b200 import synth
    from elara_b200.gpu_ops import replay_rows, ScalarTable
    n, D, K = 262_144, 64, 3
    c = synth.replay_case(n, 4_000_000, D, K, 50, 1234)
    t = {k: torch.from_numpy(v).to(dev) for k, v in c.items()}
    a = ref['gpu_ops'].replay_rows(t['rows'], t['logs'], t['offs'], t['steps'], t['cnt'], D, K, 1234, 0.01,
                                   ref['gpu_ops'].ScalarTable(*HYP, 50, dev))
    b = replay_rows(t['rows'], t['logs'], t['offs'], t['steps'], t['cnt'], D, K, 1234, 0.01, ScalarTable(*HYP, 50, dev))
    torch.cuda.synchronize()
    assert same_bits(a, b)


# ------------------------------------------------------------------------------------------------ end to end
def run_elara(ref, dev, substituted, R, C, dyn_slots, D, K, batch, steps, seed=42, L=8, depth=3):
    """One training-shaped run of the reference's planner + executor; returns the final state as a dict of tensors."""
    from elara_b200 import synth
    relara, rexec, rops = ref['elara'], ref['executor'], ref['ops']
    stock = dict(e_init=relara.init_rows, e_replay=relara.replay_rows, e_adam=relara.gpu_adam, x_init=rexec.init_rows,
                 x_replay=rexec.replay_rows, x_adam=rexec.gpu_adam, x_table=rexec.ScalarTable, dir_ext=rops.dir_ext)
    if substituted:        # the re-pointing a maintainer does (the names the reference's modules resolve at call time)
        import elara_b200.ops as b_ops
        import elara_b200.gpu_ops as b_gpu
        relara.init_rows = rexec.init_rows = b_gpu.init_rows
        relara.replay_rows = rexec.replay_rows = b_gpu.replay_rows
        relara.gpu_adam = rexec.gpu_adam = b_ops.gpu_adam
        rexec.ScalarTable = b_gpu.ScalarTable
        rops.dir_ext = b_ops.dir_ext
    try:
        sizes, offs = synth.table_sizes(R, 26, seed=seed)
        ids = [torch.from_numpy(synth.zipf_lookups(sizes, offs, batch, 1.1, seed, s + 1)).to(dev) for s in range(steps)]
        U = [torch.unique(i) for i in ids]
        # static hot set: the most frequent rows of the first ten batches
        head = torch.cat(ids[:10])
        uu, cc = torch.unique(head, return_counts=True)
        n0 = min(C - dyn_slots, uu.numel())
        static_rows = uu[torch.argsort(cc, descending=True, stable=True)[:n0]].sort().values
        bound = float(np.sqrt(1.0 / sizes.max()))
        cfg = dict(lr=HYP[0], b1=HYP[1], b2=HYP[2], eps=HYP[3], seed=seed, bound=bound, max_step=steps)
        pl = relara.ELARAPlanner(R, C, K, 'static', 'ttl', 'T', static_rows, L, dev, torch.from_numpy(offs),
                                 torch.full((26,), K, dtype=torch.int8), evict_logs=1, dir_impl='cpp')
        ex = relara.ELARAExecutor(R, D, cfg, pl, dev, threads=8, depth=depth)
        ex.load_static()
        gen = torch.Generator(device=dev).manual_seed(seed)
        for j in range(min(steps, L + 1)):
            pl.observe(j + 1, U[j])
        nxt = [0]

        def get_plan():
            s = nxt[0]
            nxt[0] += 1
            if s + L + 1 < steps:
                pl.observe(s + L + 2, U[s + L + 1])
            p = pl.plan(s + 1, U[s], [U[s + k] for k in range(1, depth) if s + k < steps])
            if p.barrier:
                ex.mark_barrier(p.s)
            return p
        ahead = collections.deque()
        for _ in range(min(steps, depth - 1)):
            ahead.append(get_plan())
            ex.enqueue_gather(ahead[-1])
        for s in range(steps):
            p = ahead.popleft()
            if s + depth - 1 < steps:
                ahead.append(get_plan())
                ex.enqueue_gather(ahead[-1])
            W, bufs = ex.assemble(p)
            gW = torch.randn(p.n, D, device=dev, generator=gen) * 1e-3
            ex.update(p, gW, bufs)
        ex.drain()
        torch.cuda.synchronize(dev)
        Kk, Lcap, Cdyn = pl.Kmax, pl.log_cap, pl.Cdyn
        nf = int(pl.n_lfree)
        ent = pl.ent[:R * Kk]
        live_ids = ent[ent >= 0].long().cpu()
        out = dict(code=pl.code, loc=pl.loc[:R], ent=ent, lstep=pl.lstep[:Lcap], lfree=pl.lfree[:nf], n_lfree=pl.n_lfree,
                   log_top=pl.log_top, mat_top=pl.mat_top, live=pl.live, adm_c0=pl.adm_c0, rj=pl.rj, pstep=pl.pstep[:Cdyn],
                   kthr=pl.kthr, toff=pl.toff, slot_of=pl.slot_of, slot_row=pl.slot_row, rok=pl.rok,
                   free=pl.free, dyn_slots=pl.dyn_slots, tcount=pl.tcount, pool=ex.pool, glog=ex.glog[:Cdyn],
                   mat=ex.store.mat[:int(pl.mat_top)].clone(), live_logs=ex.store.logs[live_ids].clone(),
                   W_last=W)
        stats = dict(pl.stats)
        ex.close()
        return out, stats
    finally:
        relara.init_rows, relara.replay_rows, relara.gpu_adam = stock['e_init'], stock['e_replay'], stock['e_adam']
        rexec.init_rows, rexec.replay_rows, rexec.gpu_adam = stock['x_init'], stock['x_replay'], stock['x_adam']
        rexec.ScalarTable, rops.dir_ext = stock['x_table'], stock['dir_ext']


def compare_runs(a, b):
    for k in a:
        x, y = a[k], b[k]
        assert x.shape == y.shape, f'{k}: shapes {tuple(x.shape)} vs {tuple(y.shape)}'
        if x.dtype == torch.float32:
            assert same_bits(x, y), f'{k} differs'
        else:
            assert torch.equal(x, y), f'{k} differs'


@pytest.mark.parametrize('case', ['middle', 'state_directory_configuration'])
def test_reference_planner_and_executor_with_this_library(dev, ref, case):
    if case == 'middle':
        args = dict(R=2_000_000, C=200_000, dyn_slots=32_768, D=128, K=3, batch=2048, steps=120)
    else:
        free, _ = torch.cuda.mem_get_info(dev)
        if free < 60 * 2**30:
            pytest.skip('needs ~50 GB of device memory')
        args = dict(R=33_800_000, C=8_000_000, dyn_slots=131_072, D=128, K=3, batch=8192, steps=100)
    stock, st_a = run_elara(ref, dev, False, **args)
    ours, st_b = run_elara(ref, dev, True, **args)
    assert st_a == st_b
    # the run exercises what it is meant to: hits, admissions, evictions back to logs, appends, compactions, replay inputs
    for key in ('hits', 'adm', 'ev', 'appends', 'compactions', 'L', 'N'):
        assert st_a[key] > 0, f'{key} never happened in this run'
    assert int(stock['live']) > 0 and int(stock['mat_top']) > 0
    compare_runs(stock, ours)
