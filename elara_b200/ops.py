"""Mirror of the reference's `srm2.ops` for the GPU hot path (reference: srm2/ops.py).

Same names, argument meaning and error behaviour; the work is done by the sm_100a kernels of
libsrm2_b200.so through its C ABI.  The host capacity-tier helpers of the reference's `ext()` (cpu_gather,
cs_append, ...) are not part of this library.
"""
import ctypes as C

import torch

from . import _lib


class _Ext:
    """Stand-in for the object returned by the reference's `ext()` (srm2/ops.py:19-26): only the part the GPU
    path uses, `adam_scalars`, is provided.  The host-tier functions stay with the reference's own extension."""

    _HOST_TIER = ('cpu_adam', 'cpu_gather', 'cpu_scatter', 'cpu_gather_var', 'cpu_scatter_slot', 'cpu_prefault',
                  'cs_gather_full', 'cs_gather_logs', 'cs_append', 'cs_write_full', 'mem_hugepage', 'mem_populate')

    @staticmethod
    def adam_scalars(lr, b1, b2, eps, step):
        """-> list of 8 floats (lr, b1, 1-b1, b2, 1-b2, 1-b1^t, 1-b2^t, eps); reference: srm2_cpu.cpp:255-257."""
        out = (C.c_float * 8)()
        _lib.check(_lib.lib().srm2_adam_scalars(lr, b1, b2, eps, int(step), out), 'adam_scalars')
        return list(out)

    def __getattr__(self, name):
        if name in self._HOST_TIER:
            raise AttributeError(f'{name} belongs to the host capacity tier, which this library does not provide; '
                                 'take it from the reference extension (srm2.ops.ext())')
        raise AttributeError(name)


_ext = _Ext()


def ext():
    return _ext


def _scalars(lr, b1, b2, eps, step):
    out = (C.c_float * 8)()
    _lib.check(_lib.lib().srm2_adam_scalars(lr, b1, b2, eps, int(step), out), 'adam_scalars')
    return out


def _require_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f'{name} must be a CUDA tensor: this library has no CPU path')


def gpu_adam(pool, slots, grad, lr, b1, b2, eps, step):
    """pool [C,3,D] cuda float32; slots int32/int64 [n] (distinct rows of pool); grad [n,D] (row i -> slots[i]).
    In place, on the current stream, no synchronisation; n == 0 is a no-op (reference: srm2/ops.py:59-67)."""
    n = slots.numel()
    if n == 0:
        return
    _require_cuda(pool, 'pool')
    if pool.dtype != torch.float32 or grad.dtype != torch.float32:
        raise TypeError('pool and grad must be float32')
    if slots.dtype not in (torch.int32, torch.int64):
        raise TypeError('slots must be int32 or int64')
    if not (pool.is_contiguous() and grad.is_contiguous() and slots.is_contiguous()):
        raise RuntimeError('pool, slots and grad must be contiguous')
    if pool.dim() != 3 or pool.shape[1] != 3:
        raise RuntimeError('pool must have shape [C,3,D]')
    D = pool.shape[2]
    if grad.numel() != n * D:
        raise RuntimeError(f'grad has {grad.numel()} elements, expected n*D = {n * D}')
    if slots.device != pool.device or grad.device != pool.device:
        raise RuntimeError('pool, slots and grad must be on the same device')
    sc = _scalars(lr, b1, b2, eps, step)
    with torch.cuda.device(pool.device):
        st = _lib.lib().srm2_adam_rows_f32(pool.data_ptr(), slots.data_ptr(), int(slots.dtype == torch.int64), grad.data_ptr(),
                                           n, D, sc, _lib.stream_of(pool.device))
    _lib.check(st, 'gpu_adam')


# ---------------------------------------------------------------------------------------------------------
# Subsystem without a function in the reference package: the driver calls torch.unique and
# aten.embedding_dense_backward directly (srm2/train.py:352, 429).  These two functions keep those calls'
# argument and return conventions, so the substitution in a driver is one line each.

_scratch_cache = {}


def _scratch(device, nbytes, tag):
    """A reusable byte buffer per (device, tag, current stream); grown when needed.  The library itself allocates nothing.
    Calls enqueued on different streams therefore never share scratch memory; calls on one stream are ordered by it."""
    key = (device, tag, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _scratch_cache[key] = buf
    return buf


def unique_inverse(ids, n_rows, sync=True, n_dev=None):
    """Sorted distinct ids and the inverse index, as `torch.unique(ids, return_inverse=True)` (srm2/train.py:352).

    ids: cuda int64 [n] in [0, n_rows) (global row ids; n_rows = total rows of all tables).
    sync=True  -> (u [n_unique], inv [n]) exactly like torch.unique (one host sync for the size, as torch does)
    sync=False -> (u_buf [min(n, n_rows)], inv [n], count) with count a cuda int64 [2] tensor
                  (count[0] = n_unique, count[1] = 1 if an id was out of range); nothing waits on the GPU.
    n_dev: optional cuda int64 [1]: only the first min(n, n_dev) lookups exist (the rest of ids / inv is ignored)."""
    _require_cuda(ids, 'ids')
    if ids.dtype != torch.int64:
        raise TypeError('ids must be int64')
    ids = ids.contiguous().reshape(-1)
    n = ids.numel()
    dev = ids.device
    cap = min(n, int(n_rows))
    L = _lib.lib()
    u = torch.empty(cap, dtype=torch.int64, device=dev)
    inv = torch.empty(n, dtype=torch.int64, device=dev)
    count = torch.empty(2, dtype=torch.int64, device=dev)
    nb = L.srm2_unique_scratch_bytes(int(n_rows))
    scr = _scratch(dev, nb, 'unique')
    with torch.cuda.device(dev):
        st = L.srm2_unique_inverse_nd_i64(_lib.ptr(ids), n, _lib.ptr(n_dev), int(n_rows), _lib.ptr(u), cap, _lib.ptr(inv),
                                          count.data_ptr(), scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'unique_inverse')
    if not sync:
        return u, inv, count
    c = count.tolist()
    if c[1]:
        raise RuntimeError(f'unique_inverse: an id lies outside [0, {n_rows})')
    return u[:c[0]], inv


def _check_grad_inv(grad, inv):
    _require_cuda(grad, 'grad')
    if grad.dtype != torch.float32 or inv.dtype != torch.int64:
        raise TypeError('grad must be float32 and inv int64')
    if grad.dim() != 2 or not grad.is_contiguous() or not inv.is_contiguous() or inv.numel() != grad.shape[0]:
        raise RuntimeError('grad must be a contiguous [n,D] tensor and inv a contiguous [n] tensor')
    if grad.shape[1] % 4:
        raise RuntimeError('segment_reduce needs D % 4 == 0')
    if inv.device != grad.device:
        raise RuntimeError('grad and inv must be on the same device')


ORDER_AUTO, ORDER_RUNS, ORDER_WINDOWS = 0, 1, 2


def segment_reduce(grad, inv, n_unique, order=ORDER_AUTO):
    """gW[j] = sum of grad[p] over lookups p with inv[p] == j, fp32, in the summation order of PyTorch's CUDA
    `aten.embedding_dense_backward(grad, inv, n_unique, -1, False)` (srm2/train.py:429) -> [n_unique, D]."""
    _check_grad_inv(grad, inv)
    n, D = grad.shape
    dev = grad.device
    out = torch.empty(int(n_unique), D, device=dev)
    if n_unique == 0:
        return out
    L = _lib.lib()
    nb = L.srm2_segment_scratch_bytes(n, int(n_unique), D)
    scr = _scratch(dev, nb, 'segment')
    with torch.cuda.device(dev):
        st = L.srm2_segment_reduce_f32(_lib.ptr(grad), _lib.ptr(inv), n, D, int(n_unique), 0, int(n_unique), order, out.data_ptr(),
                                       scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'segment_reduce')
    return out


def reduce_adam(pool, slots, grad, inv, lr, b1, b2, eps, step, n_unique=None, count=None, order=ORDER_AUTO, n_dev=None):
    """segment_reduce followed by gpu_adam(pool, slots, gW, ...) in one pass over the gradients: same bits, gW never
    materialised.  slots int64 [>= n_unique]: pool row of each unique row.  Give either n_unique (host int) or count
    (the cuda tensor returned by unique_inverse(sync=False)); with count nothing waits on the GPU."""
    _check_grad_inv(grad, inv)
    _require_cuda(pool, 'pool')
    if pool.dtype != torch.float32 or not pool.is_contiguous() or pool.dim() != 3 or pool.shape[1] != 3 or pool.shape[2] != grad.shape[1]:
        raise RuntimeError('pool must be a contiguous float32 [C,3,D] tensor with the D of grad')
    if slots.dtype != torch.int64 or not slots.is_contiguous():
        raise TypeError('slots must be a contiguous int64 tensor')
    n, D = grad.shape
    dev = grad.device
    cap = slots.numel() if n_unique is None else int(n_unique)
    if n_unique is None and count is None:
        raise RuntimeError('give n_unique or count')
    if cap > slots.numel():
        raise RuntimeError('slots is shorter than n_unique')
    if cap == 0:
        return
    L = _lib.lib()
    sc = _scalars(lr, b1, b2, eps, step)
    nb = L.srm2_segment_scratch_bytes(n, cap, D)
    scr = _scratch(dev, nb, 'segment')
    with torch.cuda.device(dev):
        st = L.srm2_reduce_adam_nd_f32(pool.data_ptr(), slots.data_ptr(), _lib.ptr(grad), _lib.ptr(inv), n, _lib.ptr(n_dev), D,
                                    -1 if n_unique is None else cap, 0 if count is None or n_unique is not None else count.data_ptr(),
                                    cap, order, sc, scr.data_ptr(), scr.numel(), _lib.stream_of(dev))
    _lib.check(st, 'reduce_adam')


def dir_ext():
    """ELARA state-directory operations (reference: srm2/ops.py:32-39): object with elara_dir_a / elara_dir_b."""
    from .directory import dir_ext as _d
    return _d()
