"""Mirror of the reference's `srm2.gpu_ops` (reference: srm2/gpu_ops.py): deterministic row initialisation and
exact replay of short gradient logs, on the sm_100a kernels of libsrm2_b200.so."""
import torch

from . import _lib
from .ops import ext


def _seed32(seed):
    # the reference kernel converts its integer seed argument to uint32 (srm2/gpu_ops.py:31-32)
    return int(seed) & 0xFFFFFFFF


def init_rows(rows, D, seed, bound, out=None):
    """rows: cuda int64 [n] -> out [n,3,D] (w0, 0, 0) (reference: srm2/gpu_ops.py:41-48)."""
    n = rows.numel()
    if not rows.is_cuda:
        raise RuntimeError('rows must be a CUDA tensor: this library has no CPU path')
    if rows.dtype != torch.int64:
        raise TypeError('rows must be int64')
    if out is None:
        out = torch.empty(n, 3, D, device=rows.device)
    if n:
        if not (out.is_contiguous() and out.dtype == torch.float32 and out.numel() == n * 3 * D and out.device == rows.device):
            raise RuntimeError('out must be a contiguous float32 [n,3,D] tensor on the device of rows')
        rows = rows.contiguous()
        with torch.cuda.device(rows.device):
            st = _lib.lib().srm2_init_rows_f32(out.data_ptr(), rows.data_ptr(), n, D, _seed32(seed), float(bound),
                                               _lib.stream_of(rows.device))
        _lib.check(st, 'init_rows')
    return out


class ScalarTable:
    """Per-logical-step Adam scalars, [max_step+1, 8] float32 with row 0 zeros (reference: srm2/gpu_ops.py:82-88)."""

    def __init__(self, lr, b1, b2, eps, max_step, device):
        e = ext()
        t = torch.tensor([e.adam_scalars(lr, b1, b2, eps, s) if s > 0 else [0.0] * 8 for s in range(max_step + 1)],
                         dtype=torch.float32)
        self.t = t.to(device)


def replay_rows(rows, logs, offs, steps, cnt, D, K, seed, bound, table, out=None):
    """rows int64 [n]; logs flat [sum(cnt),D] with row i at offs[i]; steps int32 [n,K]; cnt int32 [n] -> [n,3,D]
    (reference: srm2/gpu_ops.py:91-99)."""
    n = rows.numel()
    if not rows.is_cuda:
        raise RuntimeError('rows must be a CUDA tensor: this library has no CPU path')
    if out is None:
        out = torch.empty(n, 3, D, device=rows.device)
    if n:
        if rows.dtype != torch.int64 or offs.dtype != torch.int64 or steps.dtype != torch.int32 or cnt.dtype != torch.int32:
            raise TypeError('rows/offs must be int64, steps/cnt int32')
        if logs.dtype != torch.float32 or table.t.dtype != torch.float32:
            raise TypeError('logs and table must be float32')
        if not (out.is_contiguous() and out.dtype == torch.float32 and out.numel() == n * 3 * D and out.device == rows.device):
            raise RuntimeError('out must be a contiguous float32 [n,3,D] tensor on the device of rows')
        for name, t in (('rows', rows), ('logs', logs), ('offs', offs), ('steps', steps), ('cnt', cnt), ('table', table.t)):
            if not t.is_contiguous():
                raise RuntimeError(f'{name} must be contiguous')
            if t.device != rows.device:
                raise RuntimeError(f'{name} must be on the device of rows')
        if steps.numel() != n * K or cnt.numel() != n or offs.numel() != n:
            raise RuntimeError('steps must be [n,K], cnt and offs [n]')
        with torch.cuda.device(rows.device):
            st = _lib.lib().srm2_replay_rows_f32(out.data_ptr(), rows.data_ptr(), logs.data_ptr() if logs.numel() else table.t.data_ptr(),
                                                 offs.data_ptr(), steps.data_ptr(), cnt.data_ptr(), n, D, K, _seed32(seed),
                                                 float(bound), table.t.data_ptr(), table.t.shape[0],
                                                 _lib.stream_of(rows.device))
        _lib.check(st, 'replay_rows')
    return out
