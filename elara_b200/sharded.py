"""Row-sharded sparse Adam step: tables split by row_id mod world over the GPUs of one node.

No counterpart in the reference (it is single-GPU); this is the multi-GPU form of its sparse step
(srm2/train.py:352 unique, :429 segment-reduce, srm2/ops.py:59-67 Adam) for the row-sharded benchmark configuration.

Per step and rank:
  1. route    stable grouping of this rank's lookups by owner (row_id mod world)
  2. exchange one of three forms, chosen by enable_p2p():
              pull (default)  only the names of the lookups (local row id, source rank and position) are stored into the
                              owners' receive buffers over NVLink; the owner's fused reduce + Adam kernel then reads every
                              gradient row from the rank that produced it
              push            the routing kernel stores ids and gradient rows into the owners' receive buffers
              NCCL            all-to-all of counts, ids and gathered gradient rows (no peer access needed)
  3. update   dedup -> segment-reduce -> Adam on the local shard (fused, runs-of-10 order)
run_steps() takes a window of steps whose ids are known ahead and runs it as a pipeline of stages on separate streams
(see _run_steps_staged); step() is the plain one-step form.
Bitwise equality with a single process: ranks hold consecutive slices of the global batch, the grouping is stable and
every owner receives its lookups in rank order, so it sees the lookups of a row in ascending global position — the
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
        self.use_tma = True          # dispatch rows with bulk asynchronous copies (one warp per SM) instead of load/store threads
        if world > 1:
            n = int(max_lookups_per_rank)
            self._lid = torch.empty(n, dtype=torch.int64, device=device)
            self._grad = torch.empty(n, D, device=device)
            self._counts = torch.empty(world, dtype=torch.int64, device=device)
            self._pipe = None

    # ---- lean host path: cached pointers and preallocated buffers, two C calls per shard update --------------------
    def _fast_state(self, n_max):
        f = getattr(self, '_fast', None)
        if f is None or f['n'] < n_max:
            L = _lib.lib()
            n_rows = max(self.n_local if self.world > 1 else self.total_rows, 1)
            cap_u = min(n_max, n_rows)
            mk = lambda n, dt: torch.empty(max(n, 1), dtype=dt, device=self.dev)
            f = dict(n=n_max, n_rows=n_rows, cap_u=cap_u, u=mk(cap_u, torch.int64), inv=mk(n_max, torch.int64),
                     scr_u=mk(L.srm2_unique_scratch_bytes(n_rows), torch.uint8),
                     scr_s=mk(L.srm2_segment_scratch_bytes(n_max, cap_u, self.D), torch.uint8))
            # three sets for the staged form: dedup of step s+2, index half of step s+1 and sum half of step s each work on
            # their own (allocated on first use)
            f['u2'], f['inv2'], f['scr_s2'] = [f['u']], [f['inv']], [f['scr_s']]
            self._fast = f
        return f

    def _update_fast(self, ids_ptr, n, grad_ptr, n_dev_ptr, step, count_ptr, order, stream):
        """dedup + fused segment-reduce + Adam of n (or *n_dev) lookups on the shard; everything by address."""
        L = _lib.lib()
        f = self._fast_state(n)
        _lib.check(L.srm2_unique_inverse_nd_i64(ids_ptr, n, n_dev_ptr, f['n_rows'], f['u'].data_ptr(), f['cap_u'], f['inv'].data_ptr(),
                                                count_ptr, f['scr_u'].data_ptr(), f['scr_u'].numel(), stream), 'unique_inverse')
        sc = ops._scalars(*self.hyper, step)
        _lib.check(L.srm2_reduce_adam_nd_f32(self.pool.data_ptr(), f['u'].data_ptr(), grad_ptr, f['inv'].data_ptr(), n, n_dev_ptr, self.D,
                                             -1, count_ptr, min(n, f['cap_u']), order, sc, f['scr_s'].data_ptr(), f['scr_s'].numel(),
                                             stream), 'reduce_adam')

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
            count = torch.empty(2, dtype=torch.int64, device=self.dev)
            self._update_fast(ids.data_ptr(), ids.numel(), grads.data_ptr(), 0, step, count.data_ptr(), ops.ORDER_AUTO,
                              torch.cuda.current_stream(self.dev).cuda_stream)
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

    # ------------------------------------------------------------------------------------------------------------
    # Software-pipelined form for a sequence of steps whose inputs are known ahead (a training loop reads its batches
    # ahead of the optimizer): routing and the all-to-all of step s+1 run on a second stream while the shard update of
    # step s runs on the caller's stream; the host reads the split sizes of step s+1 while the GPU is busy with step s,
    # so the read never leaves the GPU idle.  Results are identical to calling step() in order.
    def _pipe_buffers(self, n_max):
        if self._pipe is None or self._pipe['n'] < n_max:
            cap = 2 * n_max + 1024                                  # room for an unbalanced owner
            mk = lambda *shape, dt=torch.float32: torch.empty(*shape, dtype=dt, device=self.dev)
            self._pipe = dict(n=n_max, cap=cap, comm=torch.cuda.Stream(self.dev),
                              lid=[mk(n_max, dt=torch.int64) for _ in range(2)], grad=[mk(n_max, self.D) for _ in range(2)],
                              counts=[mk(self.world, dt=torch.int64) for _ in range(2)], rcounts=[mk(self.world, dt=torch.int64) for _ in range(2)],
                              hcounts=[torch.empty(2, self.world, dtype=torch.int64).pin_memory() for _ in range(2)],
                              rlid=[mk(cap, dt=torch.int64) for _ in range(2)], rgrad=[mk(cap, self.D) for _ in range(2)])
        return self._pipe

    def run_steps(self, batches, first_step, stage_events=None):
        """batches: list of (ids, grads) of this rank, one per step; step numbers first_step, first_step+1, ...
        Returns the list of per-step count tensors (see step()).  stage_events: optional list of (start, end) CUDA events
        per step, recorded by the library around the sum half of that step (the kernels that stream the gradient rows)."""
        self._stage_events = stage_events
        import torch.distributed as dist
        if self.world == 1:
            n0 = batches[0][0].numel() if batches else 0
            if n0 <= 3072 or any(i.numel() != n0 for i, _ in batches):     # small or ragged batches: the one-call form
                return [self.step(i, g, first_step + k) for k, (i, g) in enumerate(batches)]
            return self._run_steps_staged(batches, first_step)
        if getattr(self, '_peer', None) is not None:
            return self._run_steps_p2p(batches, first_step)
        K = len(batches)
        P = self._pipe_buffers(max(i.numel() for i, _ in batches))
        comm, comp = P['comm'], torch.cuda.current_stream(self.dev)
        L = _lib.lib()
        ev_counts = [torch.cuda.Event() for _ in range(K)]
        ev_payload = [torch.cuda.Event() for _ in range(K)]
        ev_done = [torch.cuda.Event() for _ in range(K)]
        ev_start = torch.cuda.Event(); ev_start.record(comp)
        recv_n = [0] * K

        def prepare(k):                       # route + exchange of the counts, on the side stream
            ids, grads = batches[k]
            b = k & 1
            n = ids.numel()
            with torch.cuda.stream(comm):
                if k >= 2:
                    comm.wait_event(ev_done[k - 2])           # the buffers of this parity are free again
                nb = L.srm2_route_scratch_bytes(n, self.world)
                scr = ops._scratch(self.dev, nb, 'route')
                st = L.srm2_route_by_owner(_lib.ptr(ids), _lib.ptr(grads), n, self.D, self.world, P['lid'][b].data_ptr(),
                                           P['grad'][b].data_ptr(), P['counts'][b].data_ptr(), scr.data_ptr(), scr.numel(),
                                           comm.cuda_stream)
                _lib.check(st, 'route_by_owner')
                dist.all_to_all_single(P['rcounts'][b], P['counts'][b], group=self.group)
                P['hcounts'][b][0].copy_(P['counts'][b], non_blocking=True)
                P['hcounts'][b][1].copy_(P['rcounts'][b], non_blocking=True)
                ev_counts[k].record(comm)

        def payload(k):                       # needs the split sizes on the host
            b = k & 1
            n = batches[k][0].numel()
            ev_counts[k].synchronize()
            send = P['hcounts'][b][0].tolist(); recv = P['hcounts'][b][1].tolist()
            nr = int(sum(recv))
            if nr > P['cap']:
                raise RuntimeError('receive buffer too small for this batch')
            recv_n[k] = nr
            with torch.cuda.stream(comm):
                dist.all_to_all_single(P['rlid'][b][:nr], P['lid'][b][:n], output_split_sizes=recv, input_split_sizes=send, group=self.group)
                dist.all_to_all_single(P['rgrad'][b][:nr], P['grad'][b][:n], output_split_sizes=recv, input_split_sizes=send, group=self.group)
                ev_payload[k].record(comm)

        comm.wait_event(ev_start)
        prepare(0); payload(0)
        out = []
        for k in range(K):
            b = k & 1
            if k + 1 < K:
                prepare(k + 1)
            comp.wait_event(ev_payload[k])
            nr = recv_n[k]
            u, inv, count = ops.unique_inverse(P['rlid'][b][:nr], max(self.n_local, 1), sync=False)
            ops.reduce_adam(self.pool, u, P['rgrad'][b][:nr], inv, *self.hyper, first_step + k, count=count, order=ops.ORDER_RUNS)
            ev_done[k].record(comp)
            self.last_local_lookups = nr
            self.last_local_lookups_total += nr
            out.append(count)
            if k + 1 < K:
                payload(k + 1)
        return out

    # ------------------------------------------------------------------------------------------------------------
    # Exchange fused into the routing kernel: routed lookups are stored straight into the owners' receive buffers through
    # peer pointers (NVLink), see srm2_route_plan / publish / dispatch.  Nothing is read on the host: the receive buffers
    # have a fixed capacity, unused rows carry id -1 and are ignored by the shard update.
    def enable_p2p(self, max_lookups_per_rank, slack=1.5, pull=True, grad_slots=4, presum=True):
        """Allocates the symmetric buffers and exchanges their addresses.  Collective over the group.
        pull=True: only lookup names are exchanged and the owners read the gradient rows from `grad_slots` peer-visible
        gradient buffers of [max_lookups_per_rank, D] (grad_slot(k) is the one step k uses: write the gradients there to
        avoid a copy).  pull=False: the rows are stored into the owners' receive buffers.
        presum (pull only): the leading lookups of a run that come from one rank are added up by that rank and cross
        NVLink as one row (srm2_presum_*; same bits, fewer bytes); needs fewer than 2^23 lookups per rank.
        Returns True when peer access is available; otherwise the NCCL all-to-all path stays in use."""
        import ctypes as C
        import torch.distributed as dist
        if self.world == 1 or self.world > 16:
            return False
        if pull and (max_lookups_per_rank >= 1 << 24 or grad_slots < 4):
            raise ValueError('pull mode: at most 2^24-1 lookups per rank; at least four gradient slots (the exchange runs three steps ahead)')
        try:
            import torch.distributed._symmetric_memory as symm
            W, D = self.world, self.D
            n_max = int(max_lookups_per_rank)
            cap = int(n_max * slack) + 4096
            nrb = 4 if pull else 2                       # receive buffers (pull: small, and the exchange runs three steps ahead)
            rlid = symm.empty(nrb * cap, dtype=torch.int64, device=self.dev)
            cmat = symm.empty(nrb * W * W, dtype=torch.int64, device=self.dev)
            if pull:
                payload = symm.empty(nrb * cap, dtype=torch.int32, device=self.dev)            # source codes
                gbuf = symm.empty(grad_slots * n_max * D, dtype=torch.float32, device=self.dev)
            else:
                payload = symm.empty(2 * cap * D, dtype=torch.float32, device=self.dev)        # gradient rows
                gbuf = None
            sig = symm.empty(48, dtype=torch.int64, device=self.dev)       # barrier tickets: exchange | requests | prepared sums
            ts = [rlid, payload, cmat, sig] + ([gbuf] if pull else [])
            presum = bool(presum and pull and cap < (1 << 23))          # names keep one bit for "a prepared sum"
            if presum:
                # per (source, owner) pair: a source's n_max lookups make at most n_max / 2 requests in all; the owners share
                # them evenly on average (row id mod W), twice that is kept per owner; a full region costs bytes, not bits
                pcap = min(n_max // 2 + 1, max(1024, 2 * n_max // W))
                req = symm.empty(grad_slots * W * pcap * 12, dtype=torch.int32, device=self.dev)
                req_n = symm.empty(grad_slots * 16, dtype=torch.int32, device=self.dev)
                outbox = symm.empty(3 * W * pcap * D, dtype=torch.float32, device=self.dev)     # three buffers of sums (step mod 3)
                ts += [req, req_n, outbox]
            h = [symm.rendezvous(t, self.group) for t in ts]
            arr = lambda ptrs: (C.c_void_p * W)(*[int(x) for x in ptrs])
            pbytes = 4 if pull else D * 4
            peer = dict(cap=cap, n_max=n_max, pull=bool(pull), nrb=nrb, rlid=rlid, payload=payload, cmat=cmat, gbuf=gbuf, sig=sig, handles=h, ticket=0,
                        p_sig=arr([h[3].buffer_ptrs[r] for r in range(W)]),
                        p_lid=[arr([h[0].buffer_ptrs[r] + b * cap * 8 for r in range(W)]) for b in range(nrb)],
                        p_payload=[arr([h[1].buffer_ptrs[r] + b * cap * pbytes for r in range(W)]) for b in range(nrb)],
                        p_cmat=[arr([h[2].buffer_ptrs[r] + b * W * W * 8 for r in range(W)]) for b in range(nrb)],
                        counts=torch.zeros(W, dtype=torch.int64, device=self.dev), n_recv=torch.zeros(2, dtype=torch.int64, device=self.dev),
                        err=torch.zeros(1, dtype=torch.int32, device=self.dev), bar=torch.zeros(1, device=self.dev),
                        comm=torch.cuda.Stream(self.dev, priority=-1))   # routing must not queue behind the shard update
            if pull:
                peer['slots'] = grad_slots
                peer['p_gbuf'] = [arr([h[4].buffer_ptrs[r] + s * n_max * D * 4 for r in range(W)]) for s in range(grad_slots)]
            peer['presum'] = presum
            if presum:
                hr, hn, ho = h[5], h[6], h[7]
                req_n.zero_()
                peer.update(pcap=pcap, req=req, req_n=req_n, outbox=outbox,
                            req_count=torch.zeros(grad_slots * 32, dtype=torch.int32, device=self.dev),
                            presum_done=torch.zeros(1, dtype=torch.int32, device=self.dev),
                            p_sig_req=arr([h[3].buffer_ptrs[r] + 128 for r in range(W)]), p_sig_sum=arr([h[3].buffer_ptrs[r] + 256 for r in range(W)]),
                            p_req=[arr([hr.buffer_ptrs[r] + s * W * pcap * 48 for r in range(W)]) for s in range(grad_slots)],
                            p_req_n=[arr([hn.buffer_ptrs[r] + s * 64 for r in range(W)]) for s in range(grad_slots)],
                            # by step mod 3: where this rank stores what rank r asked for (its region of r's buffer of sums),
                            # and where it finds what rank r prepared for it (region r of its own buffer)
                            p_push=[arr([ho.buffer_ptrs[r] + ((b * W + self.rank) * pcap) * D * 4 for r in range(W)]) for b in range(3)],
                            p_out=[arr([outbox.data_ptr() + ((b * W + r) * pcap) * D * 4 for r in range(W)]) for b in range(3)])
            rlid.fill_(-1); cmat.zero_(); sig.zero_()
            torch.cuda.synchronize(self.dev)
            dist.barrier(group=self.group)
            self._peer = peer
            return True
        except Exception as e:                                   # no peer access on this system: keep the NCCL path
            self._peer = None
            self._peer_error = repr(e)
            return False

    barrier_timeout_ns = 5_000_000_000     # a rank whose peers do not arrive within this time flags an error and carries on

    def _barrier(self, stream_handle, n_recv_ptr=0):
        """Stream-ordered barrier across the ranks (one one-warp kernel with a bounded wait, srm2_peer_barrier).
        n_recv_ptr: the device count of received lookups of the step this barrier closes; it is set to zero when the
        exchange has failed (now or earlier), so that the step's update kernels leave the shard untouched."""
        P = self._peer
        P['ticket'] += 1
        _lib.check(_lib.lib().srm2_peer_barrier(P['p_sig'], self.rank, self.world, P['ticket'], P['err'].data_ptr(), self.barrier_timeout_ns,
                                                n_recv_ptr, stream_handle), 'peer_barrier')

    def _presum_struct(self, set_, parity, tickets):
        """srm2_presum for request set `set_` (step mod grad_slots) and buffer of sums `parity` (step mod 3), with the next ticket."""
        import ctypes as C
        P, W, D = self._peer, self.world, self.D
        pc = P['pcap']
        P['ticket'] += 1
        ps = _lib.Presum()
        ps.world, ps.rank, ps.cap, ps.timeout_ns, ps.err = W, self.rank, pc, self.barrier_timeout_ns, P['err'].data_ptr()
        ps.peer_tickets, ps.ticket = C.cast(tickets, C.c_void_p), P['ticket']
        ps.peer_req, ps.peer_req_n = C.cast(P['p_req'][set_], C.c_void_p), C.cast(P['p_req_n'][set_], C.c_void_p)
        ps.req_count = P['req_count'][set_ * 32:].data_ptr()
        ps.req, ps.req_n = P['req'][set_ * W * pc * 12:].data_ptr(), P['req_n'][set_ * 16:].data_ptr()
        ps.peer_out, ps.done = C.cast(P['p_push'][parity], C.c_void_p), P['presum_done'].data_ptr()
        return ps

    def _check_exchange(self):
        e = int(self._peer['err'].item())
        if e != 0:
            self._peer['err'].zero_()
            raise RuntimeError('exchange failed (status %d: 1 = a receive buffer overflowed, 2 = a rank did not reach a barrier in time, '
                               '4 = a copy did not complete, 8 = a request for a prepared sum named a row outside the gradient buffer)' % e)

    def grad_slot(self, k):
        """Pull mode: the peer-visible gradient buffer [max_lookups_per_rank, D] that step k reads (k mod grad_slots)."""
        P = self._peer
        s = k % P['slots']
        n_max, D = P['n_max'], self.D
        return P['gbuf'][s * n_max * D:(s + 1) * n_max * D].view(n_max, D)

    def _run_steps_p2p(self, batches, first_step):
        import torch.distributed as dist
        P, W, D = self._peer, self.world, self.D
        if P['pull']:
            return self._run_steps_staged(batches, first_step)
        cap, comm, comp = P['cap'], P['comm'], torch.cuda.current_stream(self.dev)
        L = _lib.lib()
        K = len(batches)
        ev_payload = [torch.cuda.Event() for _ in range(K)]
        ev_done = [torch.cuda.Event() for _ in range(K)]
        ev_start = torch.cuda.Event(); ev_start.record(comp)
        comm.wait_event(ev_start)

        counts_out = torch.zeros(K, 2, dtype=torch.int64, device=self.dev)
        n_max = max(i.numel() for i, _ in batches)
        scr = ops._scratch(self.dev, L.srm2_route_scratch_bytes(n_max, W), 'route')
        scr_ptr, scr_len = scr.data_ptr(), scr.numel()
        cs, ms = comm.cuda_stream, comp.cuda_stream
        counts_ptr, err_ptr = P['counts'].data_ptr(), P['err'].data_ptr()
        cmat_ptr = [P['cmat'][b * W * W:].data_ptr() for b in range(2)]
        nrecv_ptr = [P['n_recv'][b:].data_ptr() for b in range(2)]
        rl_ptr = [P['rlid'][b * cap:].data_ptr() for b in range(2)]
        rg_ptr = [P['payload'][b * cap * D:].data_ptr() for b in range(2)]
        self._fast_state(cap)

        def prepare(k):
            ids, grads = batches[k]
            b, n = k & 1, ids.numel()
            with torch.cuda.stream(comm):
                if k >= 2:
                    comm.wait_event(ev_done[k - 2])               # this parity's receive buffer has been consumed
                _lib.check(L.srm2_route_plan(ids.data_ptr(), n, W, counts_ptr, scr_ptr, scr_len, cs), 'route_plan')
                _lib.check(L.srm2_route_publish(counts_ptr, P['p_cmat'][b], self.rank, W, cs), 'route_publish')
                self._barrier(cs)                                 # count matrices complete, receive buffers free
                _lib.check(L.srm2_route_dispatch(ids.data_ptr(), grads.data_ptr(), n, D, W, self.rank, cmat_ptr[b], P['p_lid'][b],
                                                 P['p_payload'][b], cap, nrecv_ptr[b], err_ptr, int(self.use_tma), scr_ptr, scr_len, cs),
                           'route_dispatch')
                self._barrier(cs, nrecv_ptr[b])                   # every row has arrived (or nothing of this step is applied)
                ev_payload[k].record(comm)

        prepare(0)
        out = []
        for k in range(K):
            b = k & 1
            if k + 1 < K:
                prepare(k + 1)
            comp.wait_event(ev_payload[k])
            # the number of rows that arrived is known to the device only (n_recv); cap bounds it
            self._update_fast(rl_ptr[b], cap, rg_ptr[b], nrecv_ptr[b], first_step + k, counts_out[k].data_ptr(), ops.ORDER_RUNS, ms)
            ev_done[k].record(comp)
            out.append(counts_out[k])
        comp.wait_stream(comm)
        self._check_exchange()
        nr = int(P['n_recv'][(K - 1) & 1].item())
        self.last_local_lookups = nr
        self.last_local_lookups_total += nr * K
        return out

    # ------------------------------------------------------------------------------------------------------------
    # The step as a pipeline of stages on separate streams, each stage one step ahead of the next.  Only the last stage
    # needs the gradients; the others depend on the lookup ids alone, which a training loop knows ahead (prefetched batches).
    #   exchange (s+3, world > 1): plan / publish / barrier / names -> owners / barrier
    #   dedup    (s+2)           : unique rows + inverse of the (received) lookups
    #   index    (s+1)           : index half of the fused reduce: sort, boundaries, plan, run descriptors
    #   sums     (s)             : sum half: streams the gradient rows — at world > 1 from the ranks that produced them, over
    #                              NVLink — and updates the shard
    # The stages are chains of small latency-bound kernels except the last, which is bandwidth-bound and made of many
    # short-lived CTAs, so the other streams' (high-priority) kernels find room on the SMs whenever they become ready.
    # world > 1: step k's rows live in gradient slot k mod grad_slots of every rank; a batch whose gradients are not
    # already that slot is copied into it between the two barriers of its exchange (every rank has finished the sums of
    # the step that used the slot before: each rank waits for them before it enters the first barrier).
    # Buffers: receive buffers exist four times, inverse, unique rows and reduce scratch three times; each stage
    # waits for the last reader of what it overwrites.  Results are identical to calling step() in order.
    def _run_steps_staged(self, batches, first_step):
        P, W, D = getattr(self, '_peer', None), self.world, self.D
        pull = W > 1
        L = _lib.lib()
        K = len(batches)
        n_k = [i.numel() for i, _ in batches]
        n_max = max(n_k)
        comp = torch.cuda.current_stream(self.dev)
        st = getattr(self, '_stage_streams', None)
        if st is None:
            # the index stages above everything (small kernels in chains: what they need is to start at once), the sums
            # prepared at the source in between (a bandwidth-bound kernel that would otherwise hold the SMs against them),
            # the caller's stream with the run-sum kernel below (values outside the device's range are clamped)
            st = self._stage_streams = [torch.cuda.Stream(self.dev, priority=-1 if q == 4 else -3) for q in range(6)]
        xs, ds, so, ix, pr, pl = st
        xss, dss, sos, ixs, ms = xs.cuda_stream, ds.cuda_stream, so.cuda_stream, ix.cuda_stream, comp.cuda_stream
        if pull:
            if n_max > P['n_max']:
                raise RuntimeError('more lookups than max_lookups_per_rank')
            cap, S = P['cap'], P['slots']
            scr_len = (L.srm2_route_scratch_bytes(n_max, W) + 255) // 256 * 256
            scr = ops._scratch(self.dev, 2 * scr_len, 'route')        # two sets: the plan runs a step ahead of the names
            scr_ptr = scr.data_ptr()
            if 'n_recv_ring' not in P:
                P['n_recv_ring'] = torch.zeros(8, dtype=torch.int64, device=self.dev)
                P['counts2'] = torch.zeros(2 * W, dtype=torch.int64, device=self.dev)
            counts_ptr, err_ptr = P['counts2'].data_ptr(), P['err'].data_ptr()
            NRB = P['nrb']
            cmat_ptr = [P['cmat'][b * W * W:].data_ptr() for b in range(NRB)]
            nrecv_ptr = [P['n_recv_ring'][q:].data_ptr() for q in range(8)]
            rl_ptr = [P['rlid'][b * cap:].data_ptr() for b in range(NRB)]
            rs_ptr = [P['payload'][b * cap:].data_ptr() for b in range(NRB)]
            slot_ptr = [self.grad_slot(q).data_ptr() for q in range(S)]
            n = cap                                                   # bound; the count is on the device (n_recv)
        else:
            n, S, NRB = n_max, 0, 1
        f = self._fast_state(n)
        cap_u = min(n, f['cap_u'])
        NB = 4                                                        # buffer sets = stages that hold one (dedup, sort, descriptors, sums)
        while len(f['u2']) < NB:
            f['u2'].append(torch.empty_like(f['u'])); f['inv2'].append(torch.empty_like(f['inv'])); f['scr_s2'].append(torch.empty_like(f['scr_s']))
        counts_out = torch.empty(K, 2, dtype=torch.int64, device=self.dev)      # both words of every step are written by its dedup
        u_ptr = [t.data_ptr() for t in f['u2']]
        inv_ptr = [t.data_ptr() for t in f['inv2']]
        ss_ptr = [t.data_ptr() for t in f['scr_s2']]
        ss_len = f['scr_s2'][0].numel()
        su_ptr, su_len = f['scr_u'].data_ptr(), f['scr_u'].numel()
        pool_ptr = self.pool.data_ptr()

        import ctypes as C
        presum = bool(pull and P['presum'] and getattr(self, 'presum', True))
        trace = bool(getattr(self, 'trace', False))               # timing events at the stage boundaries (diagnostics)
        if not getattr(self, 'host_loop', False):
            # the same loop inside the library (srm2_staged_steps): a step is ~20 launches, and issuing them from Python takes
            # longer than running them
            import ctypes as C
            vp = lambda xs: (C.c_void_p * len(xs))(*[int(x) for x in xs])
            ring = getattr(self, '_event_ring', None)
            if ring is None:
                ring = self._event_ring = [torch.cuda.Event() for _ in range(112)]
                for e in ring:
                    e.record(comp)                                # materialise the handles
            A = _lib.Staged()
            A.K, A.first_step, A.n, A.D, A.n_rows, A.cap_u = K, first_step, n, D, f['n_rows'], f['cap_u']
            A.lr, A.b1, A.b2, A.eps = self.hyper
            A.pool, A.counts_out = pool_ptr, counts_out.data_ptr()
            keep = [vp([i.data_ptr() for i, _ in batches]), vp([g.data_ptr() for _, g in batches]),
                    (C.c_int64 * K)(*n_k), vp([xss, dss, sos, ixs, ms, pr.cuda_stream, pl.cuda_stream]), vp([e.cuda_event for e in ring])]
            A.ids, A.grads, A.n_k, A.streams, A.events = (C.cast(x, C.c_void_p) for x in keep)
            for q in range(4):
                A.u[q], A.inv[q], A.scr_s[q] = u_ptr[q], inv_ptr[q], ss_ptr[q]
            A.scr_s_bytes, A.scr_u, A.scr_u_bytes = ss_len, su_ptr, su_len
            if self._stage_events:
                cached = getattr(self, '_stage_events_handles', None)       # the same list of events window after window: keep its handles
                if cached is None or cached[0] is not self._stage_events or len(cached[1]) != 2 * len(self._stage_events):
                    cached = self._stage_events_handles = (self._stage_events, vp([e.cuda_event for pair in self._stage_events for e in pair]))
                keep.append(cached[1])
                A.stage_events = C.cast(keep[-1], C.c_void_p)
            if trace:
                tev = [torch.cuda.Event(enable_timing=True) for _ in range(K * 14)]
                t0ev = torch.cuda.Event(enable_timing=True)
                for e in tev:
                    e.record(comp)
                t0ev.record(comp)
                self.trace_origin = t0ev                          # the event the trace's microseconds count from
                keep.append(vp([e.cuda_event for e in tev]))
                A.trace_events = C.cast(keep[-1], C.c_void_p)
            A.world, A.rank = W, self.rank
            if pull:
                tk = C.c_int64(P['ticket'])
                flat = lambda lists: vp([int(x) for arr_ in lists for x in arr_])
                keep += [vp(cmat_ptr), vp(rl_ptr), vp(rs_ptr), flat(P['p_cmat']), flat(P['p_lid']), flat(P['p_payload']), vp(slot_ptr),
                         flat(P['p_gbuf']), tk]
                A.cap, A.n_recv_bufs, A.n_slots, A.timeout_ns = cap, NRB, S, self.barrier_timeout_ns
                A.route_scr, A.route_scr_bytes, A.counts, A.err, A.n_recv = scr_ptr, scr_len, counts_ptr, err_ptr, P['n_recv_ring'].data_ptr()
                (A.cmat, A.recv_lid, A.recv_src, A.peer_cmat, A.peer_lid, A.peer_src, A.slot, A.peer_slot) = (C.cast(x, C.c_void_p) for x in keep[-9:-1])
                A.peer_tickets = C.cast(P['p_sig'], C.c_void_p)
                A.ticket = C.cast(C.pointer(tk), C.c_void_p)
                if presum:
                    pc = P['pcap']
                    keep += [flat(P['p_req']), flat(P['p_req_n']), vp([P['req'][q * W * pc * 12:].data_ptr() for q in range(S)]),
                             vp([P['req_n'][q * 16:].data_ptr() for q in range(S)]), flat(P['p_push']), flat(P['p_out'])]
                    A.presum_cap = pc
                    (A.peer_req, A.peer_req_n, A.req, A.req_n, A.peer_push, A.peer_out) = (C.cast(x, C.c_void_p) for x in keep[-6:])
                    A.req_count, A.presum_done = P['req_count'].data_ptr(), P['presum_done'].data_ptr()
                    A.peer_tickets_req, A.peer_tickets_sum = C.cast(P['p_sig_req'], C.c_void_p), C.cast(P['p_sig_sum'], C.c_void_p)
            rc = L.srm2_staged_steps(C.byref(A))
            if pull:
                P['ticket'] = tk.value
            _lib.check(rc, 'staged_steps')
            if pull:
                self._check_exchange()
                nr = int(P['n_recv_ring'][(K - 1) & 7].item())
            else:
                nr = n
            if trace:      # microseconds since the start: (begin, end) of exchange, dedup, sort, descriptors, sums per step
                torch.cuda.synchronize(self.dev)
                first = 0 if pull else 1
                last = 7 if presum else 5          # ... then requests and prepared sums where they exist
                self.trace_result = [tuple((t0ev.elapsed_time(tev[k * 14 + 2 * q]) * 1e3, t0ev.elapsed_time(tev[k * 14 + 2 * q + 1]) * 1e3)
                                           for q in range(first, last)) for k in range(K)]
            self.last_local_lookups = nr
            self.last_local_lookups_total += nr * K
            return [counts_out[k] for k in range(K)]
        cnt_ptr = [counts_out.data_ptr() + 16 * k for k in range(K)]
        mkev = lambda: torch.cuda.Event(enable_timing=trace)
        ev_x, ev_d, ev_i, ev_done, ev_p = ([mkev() for _ in range(K)] for _ in range(5))
        ev_begin = {q: [mkev() for _ in range(K)] for q in 'xdis'} if trace else None
        ev_start = mkev(); ev_start.record(comp)
        for q in st:
            q.wait_event(ev_start)

        def exchange(k):
            ids, grads = batches[k]
            b, nk = k % NRB, ids.numel()
            if k >= NRB:
                xs.wait_event(ev_i[k - NRB])                      # these receive buffers have been consumed
            if k >= S:
                xs.wait_event(ev_done[k - S])                     # nobody enters the barrier while it still reads slot k mod S
            if trace:
                ev_begin['x'][k].record(xs)
            _lib.check(L.srm2_route_plan(ids.data_ptr(), nk, W, counts_ptr, scr_ptr, scr_len, xss), 'route_plan')
            _lib.check(L.srm2_route_publish(counts_ptr, P['p_cmat'][b], self.rank, W, xss), 'route_publish')
            self._barrier(xss)                                    # count matrices complete, receive buffers and slot free
            if grads.data_ptr() != slot_ptr[k % S]:
                with torch.cuda.stream(xs):
                    self.grad_slot(k)[:nk].copy_(grads, non_blocking=True)
            _lib.check(L.srm2_route_dispatch_ids(ids.data_ptr(), nk, W, self.rank, cmat_ptr[b], P['p_lid'][b], P['p_payload'][b], cap,
                                                 nrecv_ptr[k & 7], err_ptr, 0, 0, 0, scr_ptr, scr_len, xss), 'route_dispatch_ids')
            self._barrier(xss, nrecv_ptr[k & 7])                  # every name has arrived, every slot is filled (or nothing is applied)
            ev_x[k].record(xs)

        def dedup(k):
            b, q = k % NRB, k % NB
            if pull:
                ds.wait_event(ev_x[k])
            if k >= NB:
                ds.wait_event(ev_done[k - NB])                    # this buffer set has been consumed
            if trace:
                ev_begin['d'][k].record(ds)
            ids_ptr, n_dev = (rl_ptr[b], nrecv_ptr[k & 7]) if pull else (batches[k][0].data_ptr(), 0)
            _lib.check(L.srm2_unique_inverse_nd_i64(ids_ptr, n, n_dev, f['n_rows'], u_ptr[q], f['cap_u'], inv_ptr[q], cnt_ptr[k],
                                                    su_ptr, su_len, dss), 'unique_inverse')
            ev_d[k].record(ds)

        def index(k):
            b, q = k % NRB, k % NB
            ix.wait_event(ev_d[k])
            if trace:
                ev_begin['i'][k].record(ix)
            src, n_dev = (rs_ptr[b], nrecv_ptr[k & 7]) if pull else (0, 0)
            _lib.check(L.srm2_reduce_adam_index(u_ptr[q], src, inv_ptr[q], n, n_dev, D, -1, cnt_ptr[k], cap_u, 0, ss_ptr[q], ss_len, ixs),
                       'reduce_adam_index')
            if presum:                                            # requests for sums prepared at the source (set k mod S)
                ps = self._presum_struct(k % S, k % 3, P['p_sig_req'])
                _lib.check(L.srm2_presum_request(n, n_dev, D, cap_u, ss_ptr[q], ss_len, C.byref(ps), ixs), 'presum_request')
            ev_i[k].record(ix)

        def prepare_sums(k):        # sums prepared at the source: gradients of step k, no table; at most two steps ahead of the sums
            pr.wait_event(ev_i[k])
            if k >= 2:
                pr.wait_event(ev_done[k - 2])
            ps = self._presum_struct(k % S, k % 3, P['p_sig_sum'])
            _lib.check(L.srm2_presum_rows_f32(slot_ptr[k % S], batches[k][0].numel(), D, C.byref(ps), pr.cuda_stream), 'presum_rows')
            ev_p[k].record(pr)

        def sums(k):
            q = k % NB
            comp.wait_event(ev_i[k])
            if presum:
                comp.wait_event(ev_p[k])
            if trace:
                ev_begin['s'][k].record(comp)
            sc = ops._scalars(*self.hyper, first_step + k)
            if self._stage_events:
                L.srm2_stage_events(self._stage_events[k][0].cuda_event, self._stage_events[k][1].cuda_event)
            if presum:
                rc = L.srm2_reduce_adam_apply_pull_f32(pool_ptr, u_ptr[q], P['p_gbuf'][k % S], P['p_out'][k % 3], err_ptr, W, n, nrecv_ptr[k & 7], D,
                                                       -1, cnt_ptr[k], cap_u, sc, ss_ptr[q], ss_len, ms)
            elif pull:
                rc = L.srm2_reduce_adam_apply_f32(pool_ptr, u_ptr[q], 0, P['p_gbuf'][k % S], W, n, nrecv_ptr[k & 7], D, -1, cnt_ptr[k], cap_u, sc,
                                                  ss_ptr[q], ss_len, ms)
            else:
                rc = L.srm2_reduce_adam_apply_f32(pool_ptr, u_ptr[q], batches[k][1].data_ptr(), 0, 1, n, 0, D, -1, cnt_ptr[k], cap_u, sc,
                                                  ss_ptr[q], ss_len, ms)
            _lib.check(rc, 'reduce_adam_apply')
            ev_done[k].record(comp)

        # prologue, then every iteration enqueues one step of every stage, the oldest first (a stage only waits for events
        # that have been recorded by then)
        for k in range(min(2, K)):
            if pull:
                exchange(k)
        for k in range(min(2, K)):
            dedup(k)
        index(0)
        if presum:
            prepare_sums(0)
        if pull and K > 2:
            exchange(2)
        out = []
        for k in range(K):
            sums(k)
            out.append(counts_out[k])
            if k + 1 < K:
                index(k + 1)
                if presum:
                    prepare_sums(k + 1)
            if k + 2 < K:
                dedup(k + 2)
            if pull and k + 3 < K:
                exchange(k + 3)
        if self._stage_events:
            L.srm2_stage_events(None, None)
        for q in st:
            comp.wait_stream(q)
        if pull:
            self._barrier(ms)                                     # no rank returns while a peer may still read its slots
            self._check_exchange()
            nr = int(P['n_recv_ring'][(K - 1) & 7].item())
        else:
            nr = n
        if trace:      # microseconds since the start: (begin, end) of exchange, dedup, index, sums per step
            torch.cuda.synchronize(self.dev)
            us = lambda e: ev_start.elapsed_time(e) * 1e3
            ends = {'x': ev_x, 'd': ev_d, 'i': ev_i, 's': ev_done}
            self.trace_result = [tuple((us(ev_begin[q][k]), us(ends[q][k])) for q in ('xdis' if pull else 'dis')) for k in range(K)]
        self.last_local_lookups = nr
        self.last_local_lookups_total += nr * K
        return out
