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
