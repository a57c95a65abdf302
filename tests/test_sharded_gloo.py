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
