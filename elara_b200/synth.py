"""Seeded synthetic inputs with the shapes of the benchmark configurations.

They stand in for the click-log workloads the reference trains on (26 single-hot sparse fields, power-law id
frequencies); no dataset record is used or reproduced.  Everything is a pure function of (seed, step), so any
process — a test, a benchmark rank, the CPU baseline — can regenerate exactly the same arrays.
"""
import numpy as np


def _rng(seed, step=0, stream=0):
    return np.random.default_rng([int(seed), int(step), int(stream)])


# ---- row-sparse Adam on one table (1,000,000 x 16; 65,536 distinct Zipf rows per step) ------------------
def zipf_rows_without_replacement(n_rows, n_pick, alpha, seed, step, sort=True):
    """n_pick distinct row ids with P(rank r) ~ r^-alpha, drawn without replacement (Gumbel top-k);
    row id = rank - 1.  Sorted ascending by default, the order torch.unique would deliver."""
    g = _rng(seed, step, 1)
    key = -alpha * np.log(np.arange(1, n_rows + 1, dtype=np.float64)) + g.gumbel(size=n_rows)
    pick = np.argpartition(-key, n_pick - 1)[:n_pick].astype(np.int64)
    return np.sort(pick) if sort else pick[g.permutation(n_pick)]


def normal_f32(shape, scale, seed, step, stream=2):
    return (_rng(seed, step, stream).standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


# ---- exact lazy replay (4,000,000 x 64 implicit rows; histories of 1..K gradients at steps in [1,50]) ---
def replay_case(n, n_rows, D, K, max_step, seed, min_cnt=1):
    g = _rng(seed, 0, 3)
    rows = np.sort(g.choice(n_rows, size=n, replace=False)).astype(np.int64)
    cnt = g.integers(min_cnt, K + 1, size=n).astype(np.int32)
    # cnt distinct steps per row, ascending: rank random keys and keep the cnt smallest
    keys = g.random((n, max_step))
    order = np.argsort(keys, axis=1)[:, :K] + 1
    order = np.where(np.arange(K)[None, :] < cnt[:, None], order, np.iinfo(np.int32).max)
    steps = np.sort(order, axis=1)
    steps = np.where(np.arange(K)[None, :] < cnt[:, None], steps, 0).astype(np.int32)
    offs = (np.cumsum(cnt, dtype=np.int64) - cnt).astype(np.int64)
    logs = (g.standard_normal((int(cnt.sum()), D), dtype=np.float32) * np.float32(1e-3)).astype(np.float32)
    return dict(rows=rows, cnt=cnt, steps=steps, offs=offs, logs=logs)


# ---- DLRM-shaped lookups (26 tables, log-uniform vocabulary sizes, truncated power-law ids) --------------
def table_sizes(total_rows, n_tables=26, lo=4, hi=10_000_000, seed=42):
    """Vocabulary sizes exp(U(ln lo, ln hi)), rescaled to sum to total_rows (remainder on the largest)."""
    g = _rng(seed, 0, 4)
    v = np.exp(g.uniform(np.log(lo), np.log(hi), size=n_tables))
    v = np.maximum(lo, np.floor(v * (total_rows / v.sum()))).astype(np.int64)
    v[np.argmax(v)] += total_rows - v.sum()
    assert v.sum() == total_rows and v.min() >= 1
    off = np.concatenate([[0], np.cumsum(v)[:-1]]).astype(np.int64)
    return v, off


def zipf_lookups(sizes, offsets, batch, alpha, seed, step, first_sample=0):
    """Global row ids [batch*T], sample-major (lookup (b,f) at position b*T+f).  Local id = floor(x)-1 where x
    follows the continuous power law p(x) ~ x^-alpha on [1, V+1): small ids are the frequent ones.
    Sample b of a step uses its own random stream, so any slice [first_sample, first_sample+batch) of a
    global batch can be produced independently (row-sharded runs)."""
    T = len(sizes)
    g = _rng(seed, step, 5)
    # one uniform per (sample, table); advance to the slice without materialising the prefix
    if first_sample:
        g.bit_generator.advance(first_sample * T)
    u = g.random((batch, T))
    V1 = (np.asarray(sizes, np.float64) + 1.0)[None, :]
    e = 1.0 - alpha
    x = ((V1 ** e - 1.0) * u + 1.0) ** (1.0 / e)
    loc = np.minimum(np.floor(x).astype(np.int64) - 1, np.asarray(sizes)[None, :] - 1)
    loc = np.maximum(loc, 0)
    return (loc + np.asarray(offsets)[None, :]).reshape(-1)
