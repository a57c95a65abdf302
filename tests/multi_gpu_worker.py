"""Worker of tests/test_gpu_multi.py, started by torchrun with one rank per GPU: runs the row-sharded step on the GPUs
(routing kernel, NCCL all-to-all, dedup + fused reduce + Adam on every shard) and compares every shard bit for bit with
the single-process CPU oracle on the whole batch."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
HYP = (1e-3, 0.9, 0.999, 1e-8)


def main():
    rank, world, local = int(os.environ['RANK']), int(os.environ['WORLD_SIZE']), int(os.environ['LOCAL_RANK'])
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    dist.init_process_group('nccl', device_id=dev)
    from elara_b200 import synth
    from elara_b200.sharded import ShardedSparseAdam
    from oracle import oracle as O
    total_rows, D, batch = 200_000, 64, 512
    sizes, offs = synth.table_sizes(total_rows, 26, lo=4, hi=60_000, seed=3)
    eng = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                            group=dist.group.WORLD)
    eng2 = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                             group=dist.group.WORLD)
    st = O.init_rows(np.arange(total_rows), D, 42, 0.01)
    rows_updated = 0
    batches = []
    for step in (1, 2, 3):
        ids = synth.zipf_lookups(sizes, offs, batch, 1.1, 7, step, first_sample=rank * batch)
        grad = synth.normal_f32((len(ids), D), 1e-3, 7, step, stream=10 + rank)
        batches.append((torch.from_numpy(ids).to(dev), torch.from_numpy(grad).to(dev)))
        c = eng.step(batches[-1][0], batches[-1][1], step)
        rows_updated += int(c[0])
        gids = np.concatenate([synth.zipf_lookups(sizes, offs, batch, 1.1, 7, step, first_sample=r * batch) for r in range(world)])
        ggrad = np.concatenate([synth.normal_f32((batch * 26, D), 1e-3, 7, step, stream=10 + r) for r in range(world)])
        u, inv = O.unique_inverse(gids)
        O.adam_rows(st, u, O.segment_reduce(ggrad, inv, len(u)), *HYP, step)
    counts = eng2.run_steps(batches, 1)                  # the software-pipelined form must give the same shard
    eng3 = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                             group=dist.group.WORLD)
    p2p = eng3.enable_p2p(batch * 26, pull=False)        # exchange fused into the routing kernel (peer stores)
    counts3 = eng3.run_steps(batches, 1)
    # pull form: names travel, the owners read the gradient rows from the ranks that produced them.  Step 1's gradients
    # are written into its slot beforehand (no copy), the others are copied in by run_steps.
    eng4 = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                             group=dist.group.WORLD)
    pull = eng4.enable_p2p(batch * 26, pull=True, grad_slots=4)
    batches4 = list(batches)
    if pull:
        g0 = eng4.grad_slot(0)[:batches[0][1].shape[0]]
        g0.copy_(batches[0][1])
        batches4[0] = (batches[0][0], g0)
    counts4 = eng4.run_steps(batches4, 1)
    eng5 = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                             group=dist.group.WORLD)
    eng5.enable_p2p(batch * 26, pull=True, grad_slots=5)
    eng5.host_loop = True                                # the same stages issued from Python instead of srm2_staged_steps
    counts5 = eng5.run_steps(batches[:2], 1) + eng5.run_steps(batches[2:], 3)
    # the pull form without sums prepared at the source (every lookup's row crosses on its own)
    eng6 = ShardedSparseAdam(total_rows, D, world, rank, dev, seed=42, bound=0.01, hyper=HYP, max_lookups_per_rank=batch * 26,
                             group=dist.group.WORLD)
    eng6.enable_p2p(batch * 26, pull=True, grad_slots=4, presum=False)
    counts6 = eng6.run_steps(batches, 1)
    torch.cuda.synchronize(dev)
    ok6 = torch.equal(eng.pool.view(torch.int32), eng6.pool.view(torch.int32)) and sum(int(c[0]) for c in counts6) == rows_updated
    shard = eng.pool.cpu().numpy()
    ok = np.array_equal(shard.view(np.uint32), st[rank::world].view(np.uint32))
    ok = ok and torch.equal(eng.pool.view(torch.int32), eng2.pool.view(torch.int32)) and sum(int(c[0]) for c in counts) == rows_updated
    ok = ok and torch.equal(eng.pool.view(torch.int32), eng3.pool.view(torch.int32)) and sum(int(c[0]) for c in counts3) == rows_updated
    ok = ok and torch.equal(eng.pool.view(torch.int32), eng4.pool.view(torch.int32)) and sum(int(c[0]) for c in counts4) == rows_updated
    ok = ok and torch.equal(eng.pool.view(torch.int32), eng5.pool.view(torch.int32)) and sum(int(c[0]) for c in counts5) == rows_updated
    # a longer window: every buffer set of the pipeline (gradient slots, request sets, both buffers of sums) is used again
    more = []
    for step in range(4, 16):
        ids = synth.zipf_lookups(sizes, offs, batch, 1.1, 7, step, first_sample=rank * batch)
        grad = synth.normal_f32((len(ids), D), 1e-3, 7, step, stream=10 + rank)
        more.append((torch.from_numpy(ids).to(dev), torch.from_numpy(grad).to(dev)))
    eng2.run_steps(more, 4); eng4.run_steps(more, 4); eng6.run_steps(more[:5], 4); eng6.run_steps(more[5:], 9)
    torch.cuda.synchronize(dev)
    ok6 = ok6 and torch.equal(eng2.pool.view(torch.int32), eng4.pool.view(torch.int32)) and torch.equal(eng2.pool.view(torch.int32), eng6.pool.view(torch.int32))
    if not (ok and ok6):
        print(f'rank {rank}: three-step checks {int(ok)}, prepared sums on/off and the longer window {int(ok6)}', flush=True)
    ok = ok and ok6
    flag = torch.tensor([int(ok), rows_updated], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f'MULTI_GPU_RESULT ok={int(flag[0])} world={world} rows_updated_min={int(flag[1])} p2p={int(p2p)} pull={int(pull)} '
              f'{getattr(eng3, "_peer_error", "")}', flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == '__main__':
    main()
