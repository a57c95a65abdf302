"""Capacity-tier record arenas in device memory (reference: ArenaStore, srm2/elara.py:40-103, and the host copies
cpu_gather / cpu_scatter / cpu_adam it is driven with, srm2/csrc/srm2_cpu.cpp:22-81).

The reference keeps MAT records [Mcap+1, 3, D] and log entries [Lcap+1, 1, D] in host DRAM and moves them by physical id.
`HbmArenaStore` holds the same two arenas, same shapes and the same trash rows, in HBM; its gather / scatter / adam take
the planner's physical ids exactly as the reference's host calls do (`S_slot`, `F_slot`, `L_ids`, `A_ids`, `W_slot`,
`EVL_ids` of a plan) and run as kernels on the current stream — no pinned staging, no host worker.  Bookkeeping
(`set_tops`, `footprint`, `resident_bytes`, the enforced budget) mirrors the reference's; there is nothing to pre-fault.
"""
import torch

from . import _lib, ops


class HbmArenaStore:
    kind = 'arena'

    def __init__(self, R, D, device, budget_bytes=0, mat_cap=None, log_cap=None):
        self.R, self.D, self.dev, self.budget = R, D, device, budget_bytes
        self.mat_cap = mat_cap or R
        self.log_cap = log_cap or 2 * R
        need = ((self.mat_cap + 1) * 3 + (self.log_cap + 1)) * D * 4
        if budget_bytes and need > budget_bytes:
            raise MemoryError(f'arenas of {need / 2**30:.1f} GiB exceed the budget of {budget_bytes / 2**30:.1f} GiB')
        self.mat = torch.empty(self.mat_cap + 1, 3, D, device=device)       # last rows = trash, as in the reference
        self.logs = torch.empty(self.log_cap + 1, 1, D, device=device)
        self.top = {'mat': 0, 'log': 0}
        self.live_logs = 0
        self._bad = torch.zeros(1, dtype=torch.int32, device=device)

    def _arena(self, which):
        return self.mat if which == 'mat' else self.logs

    def gather(self, which, ids, ncomp, out=None):
        """out[i] = the first ncomp D-vectors of record ids[i] (cpu_gather's contract); ids cuda int64."""
        a = self._arena(which)
        n, W = ids.numel(), a.shape[1]
        if out is None:
            out = torch.empty(n, ncomp, self.D, device=self.dev)
        if n:
            if ids.dtype != torch.int64 or not ids.is_contiguous() or not out.is_contiguous() or out.numel() != n * ncomp * self.D:
                raise RuntimeError('ids must be a contiguous int64 tensor and out a contiguous [n, ncomp, D] tensor')
            with torch.cuda.device(self.dev):
                st = _lib.lib().srm2_arena_gather_f32(out.data_ptr(), a.data_ptr(), ids.data_ptr(), n, a.shape[0], W, ncomp, self.D,
                                                      self._bad.data_ptr(), _lib.stream_of(self.dev))
            _lib.check(st, 'arena_gather')
        return out

    def scatter(self, which, ids, src):
        """The first Wc D-vectors of record ids[i] = src[i] (cpu_scatter's contract; src [n, Wc, D] or [n, D]); ids distinct."""
        a = self._arena(which)
        n, W = ids.numel(), a.shape[1]
        if n == 0:
            return
        Wc = src.shape[1] if src.dim() == 3 else 1
        if ids.dtype != torch.int64 or not ids.is_contiguous() or not src.is_contiguous() or src.numel() != n * Wc * self.D:
            raise RuntimeError('ids must be a contiguous int64 tensor and src a contiguous [n, Wc, D] tensor')
        with torch.cuda.device(self.dev):
            st = _lib.lib().srm2_arena_scatter_f32(a.data_ptr(), src.data_ptr(), ids.data_ptr(), n, a.shape[0], W, Wc, self.D,
                                                   self._bad.data_ptr(), _lib.stream_of(self.dev))
        _lib.check(st, 'arena_scatter')

    def adam(self, slots, grad, lr, b1, b2, eps, step):
        """Row-sparse Adam on MAT records by physical id (the reference's cpu_adam on st.mat, srm2/elara.py:567)."""
        ops.gpu_adam(self.mat, slots, grad, lr, b1, b2, eps, step)

    def bad_ids_seen(self):
        """True if a gather or scatter met an id outside its arena since the last call (synchronises)."""
        b = bool(self._bad.item())
        self._bad.zero_()
        return b

    # ---- bookkeeping, as the reference's ----
    def set_tops(self, mat_top, log_top, live_logs):
        self.top['mat'], self.top['log'], self.live_logs = mat_top, log_top, live_logs

    def resident_bytes(self):
        return (self.mat.numel() + self.logs.numel()) * 4

    def fault(self, which, upto, background=False):
        return False                                           # device memory is there from the start

    def footprint(self):
        D = self.D
        return {'store': 'elara_arena_hbm', 'mat_rows': int(self.top['mat']), 'live_log_entries': int(self.live_logs),
                'log_arena_entries': int(self.top['log']),
                'store_bytes': int(self.top['mat'] * 3 * D * 4 + self.live_logs * D * 4),
                'mat_bytes': int(self.top['mat'] * 3 * D * 4), 'log_bytes': int(self.live_logs * D * 4),
                'index_bytes': 0, 'resident_bytes': int(self.resident_bytes())}
