"""Row-sharded sparse Adam step: tables split by row_id mod world over the GPUs of one node.

No counterpart in the reference (it is single-GPU); this is the multi-GPU form of its sparse step
(srm2/train.py:352 unique, :429 segment-reduce, srm2/ops.py:59-67 Adam) for the row-sharded benchmark configuration.

Per step and rank:
  1. route    stable grouping of this rank's lookups by owner (row_id mod world) + gather of their gradient rows
  2. exchange NCCL all-to-all over NVLink: lookup counts, then local row ids and gradient rows
  3. update   dedup -> segment-reduce -> Adam on the local shard (fused, runs-of-10 order)
Bitwise equality with a single process: ranks hold consecutive slices of the global batch, the grouping is stable and
the all-to-all concatenates in rank order, so an owner sees the lookups of a row in ascending global position — the
order the single-process segment-reduce uses — and it sees all of them, so the runs of 10 are cut identically.
"""
import torch

from . import _lib, ops
from .gpu_ops import init_rows

CHUNK = 1 << 20


def exchange(lids, grads, send_counts, group, world):
    """All-to-all of the routed lookups.  lids [n] int64 and grads [n,D], grouped by destination rank with
    send_counts[d] entries for rank d (a host list).  Returns (recv_lids, recv_grads, recv_counts): what every rank
    sent to this one, concatenated in source-rank order.  Works on any backend (NCCL on GPUs; gloo in the CPU tests)."""
    import torch.distributed as dist
    dev = lids.device
    sc = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    rc = torch.empty(world, dtype=torch.int64, device=dev)
    dist.all_to_all_single(rc, sc, group=group)
    recv_counts = rc.tolist()
    n_recv = int(sum(recv_counts))
    recv_lids = torch.empty(n_recv, dtype=torch.int64, device=dev)
    recv_grads = torch.empty(n_recv, grads.shape[1], dtype=grads.dtype, device=dev)
    dist.all_to_all_single(recv_lids, lids, output_split_sizes=recv_counts, input_split_sizes=list(send_counts), group=group)
    dist.all_to_all_single(recv_grads, grads, output_split_sizes=recv_counts, input_split_sizes=list(send_counts), group=group)
    return recv_lids, recv_grads, recv_counts


def local_rows(total_rows, world, rank):
    """Number of rows with row_id mod world == rank."""
    return (total_rows - rank + world - 1) // world if total_rows > rank else 0


class ShardedSparseAdam:
    """One rank's shard [local_rows, 3, D] of the tables and the per-step pipeline."""

    def __init__(self, total_rows, D, world, rank, device, seed, bound, hyper, max_lookups_per_rank, group=None):
        self.total_rows, self.D, self.world, self.rank, self.dev = int(total_rows), D, world, rank, device
        self.hyper = tuple(hyper)
        self.group = group
        self.n_local = local_rows(self.total_rows, world, rank)
        _lib.lib()                                              # fail now if the kernels are missing
        self.pool = torch.empty(self.n_local, 3, D, device=device)
        for c in range(0, self.n_local, CHUNK):                 # counter-hash init of the global row ids this rank owns
            l = torch.arange(c, min(self.n_local, c + CHUNK), device=device)
            init_rows(l * world + rank, D, seed, bound, out=self.pool[c:c + l.numel()])
        self.last_local_lookups = 0
        self.last_local_lookups_total = 0
        if world > 1:
            n = int(max_lookups_per_rank)
            self._lid = torch.empty(n, dtype=torch.int64, device=device)
            self._grad = torch.empty(n, D, device=device)
            self._counts = torch.empty(world, dtype=torch.int64, device=device)

    def route(self, ids, grads):
        """-> (lids grouped by owner, gradient rows in the same order, per-owner counts on the device)."""
        n = ids.numel()
        L = _lib.lib()
        if n > self._lid.numel():
            raise RuntimeError('more lookups than max_lookups_per_rank')
        nb = L.srm2_route_scratch_bytes(n, self.world)
        scr = ops._scratch(self.dev, nb, 'route')
        with torch.cuda.device(self.dev):
            st = L.srm2_route_by_owner(_lib.ptr(ids), _lib.ptr(grads), n, self.D, self.world, self._lid.data_ptr(),
                                       self._grad.data_ptr(), self._counts.data_ptr(), scr.data_ptr(), scr.numel(),
                                       _lib.stream_of(self.dev))
        _lib.check(st, 'route_by_owner')
        return self._lid[:n], self._grad[:n], self._counts

    def step(self, ids, grads, step, defer=False):
        """ids int64 [n] global row ids of this rank's slice of the batch, grads [n,D].  Returns the cuda int64 [2]
        count tensor of the local dedup (count[0] = rows updated on this rank).  Nothing waits on the GPU when
        world == 1; with world > 1 the all-to-all split sizes are read on the host once per step."""
        if self.world == 1:
            u, inv, count = ops.unique_inverse(ids, self.total_rows, sync=False)
            ops.reduce_adam(self.pool, u, grads, inv, *self.hyper, step, count=count)
            self.last_local_lookups = ids.numel()
            self.last_local_lookups_total += ids.numel()
            return count
        lids, g, counts = self.route(ids, grads)
        recv_lids, recv_grads, _ = exchange(lids, g, counts.tolist(), self.group, self.world)
        u, inv, count = ops.unique_inverse(recv_lids, max(self.n_local, 1), sync=False)
        # the order is that of the whole batch: runs of 10 (the global batch is far above the small-input limit)
        ops.reduce_adam(self.pool, u, recv_grads, inv, *self.hyper, step, count=count, order=ops.ORDER_RUNS)
        self.last_local_lookups = recv_lids.numel()
        self.last_local_lookups_total += recv_lids.numel()
        return count
