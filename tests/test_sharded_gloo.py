"""Host-side logic of the row-sharded step on CPU ranks (gloo, world_size 2 and 3): stable routing + all-to-all in rank
order delivers every row's lookups to its owner in ascending global position, so the per-owner reduce + Adam equals
the single-process result bit for bit.  The device kernels are replaced here by the oracle (test-side only)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
HYP = (1e-3, 0.9, 0.999, 1e-8)


def _free_port():
    s = socket.socket(); s.bind(('127.0.0.1', 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, total_rows, D, batch, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ['MASTER_ADDR'] = '127.0.0.1'; os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    from elara_b200 import synth
    from elara_b200.sharded import exchange, local_rows
    from oracle import oracle as O
    sizes, offs = synth.table_sizes(total_rows, 26, lo=4, hi=total_rows // 3, seed=3)
    n_loc = local_rows(total_rows, world, rank)
    st = O.init_rows(np.arange(n_loc) * world + rank, D, 42, 0.01)
    for step in (1, 2, 3):
        ids = synth.zipf_lookups(sizes, offs, batch, 1.1, 7, step, first_sample=rank * batch)
        grad = synth.normal_f32((ids.shape[0], D), 1e-3, 7, step, stream=10 + rank)
        owner = ids % world
        perm = np.argsort(owner, kind='stable')                     # what srm2_route_by_owner computes on the device
        counts = np.bincount(owner, minlength=world).tolist()
        rl, rg, rc = exchange(torch.from_numpy(ids[perm] // world), torch.from_numpy(grad[perm]), counts, None, world)
        assert sum(rc) == rl.numel()
        u, inv = O.unique_inverse(rl.numpy())
        O.adam_rows(st, u, O.segment_reduce(rg.numpy(), inv, len(u), chunk=10, window=0), *HYP, step)
    np.save(Path(out_dir) / f'shard{rank}.npy', st)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 3])
def test_sharded_equals_single_process(tmp_path, oracle, world):
    from elara_b200 import synth
    from elara_b200.sharded import local_rows
    total_rows, D, batch = 5000, 16, 160
    mp.spawn(_worker, args=(world, _free_port(), total_rows, D, batch, str(tmp_path)), nprocs=world, join=True)
    # single process on the whole batch
    sizes, offs = synth.table_sizes(total_rows, 26, lo=4, hi=total_rows // 3, seed=3)
    st = oracle.init_rows(np.arange(total_rows), D, 42, 0.01)
    for step in (1, 2, 3):
        ids = np.concatenate([synth.zipf_lookups(sizes, offs, batch, 1.1, 7, step, first_sample=r * batch) for r in range(world)])
        grad = np.concatenate([synth.normal_f32((batch * 26, D), 1e-3, 7, step, stream=10 + r) for r in range(world)])
        assert len(ids) > 3072                                   # the whole batch is in the runs-of-10 regime
        u, inv = oracle.unique_inverse(ids)
        oracle.adam_rows(st, u, oracle.segment_reduce(grad, inv, len(u)), *HYP, step)
    touched = 0
    for r in range(world):
        shard = np.load(tmp_path / f'shard{r}.npy')
        assert shard.shape[0] == local_rows(total_rows, world, r)
        assert np.array_equal(shard.view(np.uint32), st[r::world].view(np.uint32))
        touched += int((shard[:, 1] != 0).any(axis=1).sum())
    assert touched > 500


@pytest.mark.parametrize('world', [2, 3, 8])
def test_sums_prepared_at_the_source_are_the_owner_s_sums(oracle, world):
    """The rule the multi-GPU exchange relies on, checked on the CPU with the oracle's arithmetic: in the order of the
    segment-reduce (lookups of a row in ascending global position, runs of ten summed from +0, run sums added from +0) the
    leading lookups of a run that come from one rank may be replaced by their own left-to-right sum from +0 — the row sums
    keep their bits.  Replacing a group further back in a run would not (shown on the same data)."""
    rng = np.random.default_rng(world)
    R, D, n = 400, 8, 6000
    p = np.arange(1, R + 1, dtype=np.float64) ** -1.1
    ids = [rng.choice(R, size=n, p=p / p.sum()).astype(np.int64) for _ in range(world)]           # rank r holds lookups r*n .. (r+1)*n-1
    grads = [(rng.standard_normal((n, D)) * 10.0 ** rng.integers(-4, 5, size=(n, 1))).astype(np.float32) for _ in range(world)]
    all_ids, all_grads = np.concatenate(ids), np.concatenate(grads)
    u, inv = oracle.unique_inverse(all_ids)
    want = oracle.segment_reduce(all_grads, inv, len(u), chunk=oracle.SEGMENT_CHUNK)
    src = np.repeat(np.arange(world), n)

    def sum_from_zero(rows):
        acc = np.zeros(D, np.float32)
        for r in rows:
            acc = (acc + all_grads[r]).astype(np.float32)
        return acc

    def reduce_with_groups(leading_only):
        out = np.zeros((len(u), D), np.float32)
        order = np.argsort(inv, kind='stable')
        bounds = np.searchsorted(inv[order], np.arange(len(u) + 1))
        replaced = 0
        for j in range(len(u)):
            pos = order[bounds[j]:bounds[j + 1]]
            total = np.zeros(D, np.float32)
            for s0 in range(0, len(pos), 10):
                run = pos[s0:s0 + 10]
                g = 0 if leading_only else next((q for q in range(1, len(run)) if src[run[q]] != src[run[q - 1]]), 0)
                m = g + 1
                while m < len(run) and src[run[m]] == src[run[g]]:
                    m += 1
                acc = np.zeros(D, np.float32)
                for q in range(g):
                    acc = (acc + all_grads[run[q]]).astype(np.float32)
                if m - g >= 2:
                    acc = (acc + sum_from_zero(run[g:m])).astype(np.float32)          # the group arrives as one row
                    replaced += m - g
                else:
                    m = g
                for q in range(m, len(run)):
                    acc = (acc + all_grads[run[q]]).astype(np.float32)
                total = (total + acc).astype(np.float32)
            out[j] = total
        return out, replaced

    got, replaced = reduce_with_groups(leading_only=True)
    assert replaced > 0.3 * len(all_ids)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    other, replaced2 = reduce_with_groups(leading_only=False)
    assert replaced2 > 0 and not np.array_equal(other.view(np.uint32), want.view(np.uint32))
