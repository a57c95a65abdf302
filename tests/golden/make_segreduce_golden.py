"""Known-answer vectors for the segment-reduce, produced by PyTorch's own CUDA operator on a GPU box.

The reference sums per-lookup gradients with `torch.ops.aten.embedding_dense_backward` (srm2/train.py:429);
the order of the fp32 additions is that operator's.  This script runs the operator (black box: inputs in,
outputs out) on inputs whose sums depend on the association order, stores inputs and outputs, and reports
which candidate order of the CPU oracle reproduces each case.

    python tests/golden/make_segreduce_golden.py [--out tests/golden/segreduce_cuda.npz]

Needs a CUDA device; the torch version that produced the committed file is stored inside it.
"""
import argparse
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))


def case(rng, n, D, n_keys, zipf=False):
    """Order-sensitive values: normal numbers over seven decades, a few zeros and negative zeros."""
    if zipf:
        p = np.arange(1, n_keys + 1, dtype=np.float64) ** -1.1
        p /= p.sum()
        keys = rng.choice(n_keys, size=n, p=p)
    else:
        keys = rng.integers(0, n_keys, n)
    _, inv = np.unique(keys, return_inverse=True)            # every index in [0, n_unique) occurs
    inv = inv.reshape(-1).astype(np.int64)
    grad = (rng.standard_normal((n, D)) * 10.0 ** rng.integers(-3, 4, (n, 1))).astype(np.float32)
    grad[rng.random(n) < 0.02] = 0.0
    grad[rng.random(n) < 0.02] = -0.0
    return grad, inv, int(inv.max()) + 1 if n else 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--out', default=str(ROOT / 'tests/golden/segreduce_cuda.npz'))
    a = ap.parse_args()
    from oracle import oracle as O
    dev = torch.device('cuda:0')
    rng = np.random.default_rng(2024)
    save = {'torch_version': np.array(torch.__version__), 'device': np.array(torch.cuda.get_device_name(0))}
    specs = []
    for n in (1, 5, 31, 32, 33, 64, 100, 767, 768, 769, 1000, 3071, 3072, 3073, 4000, 5000):
        D = 16 if n <= 1000 else 8                      # narrow rows keep the committed file small
        specs += [(n, D, 3, False), (n, D, 40, False)]
        if n <= 100 or n == 768:
            specs.append((n, 128, 7, False))
    specs += [(20000, 4, 600, True), (12000, 8, 1500, True), (4000, 32, 50, True), (3500, 24, 11, False), (3500, 12, 11, False)]
    summary = {}
    for ci, (n, D, nk, zipf) in enumerate(specs):
        grad, inv, nu = case(rng, n, D, nk, zipf)
        g_d, i_d = torch.from_numpy(grad).to(dev), torch.from_numpy(inv).to(dev)
        # default mode, several runs: for inputs above a few thousand lookups that map to FEW unique rows the operator
        # is not run-to-run deterministic in its default mode; such cases are stored with the output of
        # torch.use_deterministic_algorithms(True) and flagged.
        torch.use_deterministic_algorithms(False)
        runs = [torch.ops.aten.embedding_dense_backward(g_d, i_d, nu, -1, False).cpu().numpy() for _ in range(5)]
        stable = len({r.tobytes() for r in runs}) == 1
        torch.use_deterministic_algorithms(True)
        det = torch.ops.aten.embedding_dense_backward(g_d, i_d, nu, -1, False).cpu().numpy()
        torch.use_deterministic_algorithms(False)
        if stable:
            assert np.array_equal(det.view(np.uint32), runs[0].view(np.uint32)), 'deterministic mode differs from a stable default mode'
        out = runs[0] if stable else det
        cands = {'sequential': O.segment_reduce(grad, inv, nu, chunk=0, window=0), 'chunk10': O.segment_reduce(grad, inv, nu, chunk=10, window=0),
                 'window32': O.segment_reduce(grad, inv, nu, window=32), 'default': O.segment_reduce(grad, inv, nu)}
        match = [k for k, v in cands.items() if np.array_equal(v.view(np.uint32), out.view(np.uint32))]
        summary[(n, D, nk)] = match
        print(f'n={n:6d} D={D:4d} keys={nu:5d} zipf={int(zipf)} default-mode-stable={int(stable)} matches={match}', flush=True)
        save[f'c{ci}_grad'] = grad; save[f'c{ci}_inv'] = inv; save[f'c{ci}_nu'] = np.array(nu); save[f'c{ci}_out'] = out
        save[f'c{ci}_default_mode_stable'] = np.array(stable)
    save['n_cases'] = np.array(len(specs))
    Path(a.out).parent.mkdir(parents=True, exist_ok=True)
    np.savez_compressed(a.out, **save)
    bad = [k for k, v in summary.items() if 'default' not in v]
    print('cases not matched by the oracle default order:', bad)


if __name__ == '__main__':
    main()
