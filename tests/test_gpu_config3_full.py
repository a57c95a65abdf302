"""The DLRM-shaped sparse step at its stated size: 26 fp32 tables, d = 128, 33.8 M rows (51.9 GB of w, m, v on the GPU),
8192 x 26 Zipf(1.1) lookups per step, 100 steps of dedup -> segment-reduce -> Adam (reference: srm2/train.py:352,
425-440 and srm2/ops.py:59-67).

The engine runs the 100 steps through run_steps(), the pipelined path the benchmark times.  The oracle keeps only the
rows the 100 batches touch (a compacted table whose rows start from the counter-hash initialisation, as implicit rows
do in the reference) and applies unique -> runs-of-10 segment sums -> Adam to them on the CPU.  Every touched row must
come out bit-identical, and a large sample of untouched rows must still hold its initial record.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HYP = (1e-3, 0.9, 0.999, 1e-8)


def test_hundred_steps_on_the_33_8M_row_table(oracle):
    from elara_b200 import synth
    from elara_b200.gpu_ops import init_rows
    from elara_b200.sharded import ShardedSparseAdam
    if not torch.cuda.is_available():
        pytest.skip('needs a CUDA device')
    dev = torch.device('cuda:0')
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 62 * 2**30:
        pytest.skip('needs ~56 GB of device memory')
    R, D, B, T, steps, seed = 33_800_000, 128, 8192, 26, 100, 42
    n = B * T
    sizes, offs = synth.table_sizes(R, T, seed=seed)
    bound = float(np.sqrt(1.0 / sizes.max()))
    eng = ShardedSparseAdam(R, D, 1, 0, dev, seed=seed, bound=bound, hyper=HYP, max_lookups_per_rank=n)
    ids_np = [synth.zipf_lookups(sizes, offs, B, 1.1, seed, s + 1) for s in range(steps)]
    ids_dev = [torch.from_numpy(x).to(dev) for x in ids_np]
    gen = torch.Generator(device=dev).manual_seed(seed)
    grads_dev = [torch.randn(n, D, device=dev, generator=gen) * 1e-3 for _ in range(4)]
    grads_np = [g.cpu().numpy() for g in grads_dev]
    counts = eng.run_steps([(ids_dev[s], grads_dev[s % 4]) for s in range(steps)], 1)
    torch.cuda.synchronize(dev)

    touched = np.unique(np.concatenate(ids_np))
    state = oracle.init_rows(touched, D, seed, bound)                      # compacted table: row j <-> touched[j]
    for s in range(steps):
        u, inv = oracle.unique_inverse(ids_np[s])
        gW = oracle.segment_reduce(grads_np[s % 4], inv, len(u))           # n > 3072: runs of 10
        oracle.adam_rows(state, np.searchsorted(touched, u), gW, *HYP, s + 1, nthreads=8)
        assert int(counts[s][0]) == len(u) and int(counts[s][1]) == 0
    got = eng.pool[torch.from_numpy(touched).to(dev)].cpu().numpy()
    assert touched.shape[0] > 1_000_000
    assert np.array_equal(got.view(np.uint32), state.view(np.uint32)), 'a touched row differs from the oracle'

    rng = np.random.default_rng(1)
    cand = np.unique(rng.integers(0, R, 1_200_000))
    untouched = cand[~np.isin(cand, touched)][:1_000_000]
    rows = torch.from_numpy(untouched).to(dev)
    assert torch.equal(eng.pool[rows].view(torch.int32), init_rows(rows, D, seed, bound).view(torch.int32)), 'an untouched row changed'
