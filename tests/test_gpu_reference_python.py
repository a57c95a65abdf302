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
def ref(dev):
    """The reference's srm2 package with its two compiled extensions already loaded (no JIT build on the box)."""
    from oracle.ref_pipeline import load_reference
    r = load_reference()
    if r is None:
        pytest.skip('oracle/_ref is not staged (python oracle/build_ref.py --ref <reference checkout>)')
    return r


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
from oracle.ref_pipeline import run_elara as _run_elara


def run_elara(*args, **kw):
    out, stats = _run_elara(*args, **kw)
    stats.pop('ms_per_step', None); stats.pop('plan_ms_per_step', None)      # the timings are for the benchmark, not part of the comparison
    stats.pop('syncs', None)                  # the fused plan() reads the host less often
    return out, stats


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


def test_fused_executor_glue_under_the_reference_pipeline(dev, ref):
    """The executor's GPU glue replaced as well: assemble() through the fused assemble kernel and update() through the three
    update kernels (srm2/elara.py:479-489, 497-532), everything else the reference's own code.  Same final state, bit for
    bit, as the stock run — with and without recorded resident histories."""
    args = dict(R=2_000_000, C=200_000, dyn_slots=32_768, D=128, K=3, batch=2048, steps=120)
    stock, st_a = run_elara(ref, dev, False, **args)
    fused, st_b = run_elara(ref, dev, True, fused_executor=True, **args)
    assert st_a == st_b
    compare_runs(stock, fused)
    # ... and with the planner's plan() on the fused kernels too: nothing of the reference's GPU code is left on the step
    fused2, st_c = run_elara(ref, dev, True, fused_executor=True, fused_plan=True, **args)
    assert st_a == st_c
    compare_runs(stock, fused2)
