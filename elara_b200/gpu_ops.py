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


def assemble(n, D, pool, hit_pos, hit_slot, N_pos, N_row, L_pos, L_row, logs, L_off, L_steps, L_cnt, K, seed, bound, table,
             ff, F_pos, sw, S_pos, allow_separate_calls=False, inv=None, emb_out=None):
    """The working matrix of a step in one kernel (reference: the body of ELARAExecutor.assemble, srm2/elara.py:479-489).
    Returns (W [n,D], fullN [n_N,3,D] or None, fullL [n_L,3,D] or None) — the reference returns W, (fullN, fullL, ff).
    Index tensors are cuda int64; any of the five groups may be empty (pass empty tensors).
    inv (cuda int64 [n_lookups]) given: the forward gather of the step, emb[p] = W[inv[p]] (srm2/train.py:427), is enqueued
    right behind the assemble kernel (into emb_out [n_lookups, D] when given) and (W, fullN, fullL, emb) is returned.
    The fused kernel needs D % 4 == 0, K <= 8 and 16-byte aligned buffers.  Other shapes raise, unless
    allow_separate_calls=True asks for the same result from init_rows / replay_rows and index copies."""
    dev = pool.device
    if not pool.is_cuda:
        raise RuntimeError('pool must be a CUDA tensor: this library has no CPU path')
    W = torch.empty(n, D, device=dev)
    nh, nN, nL, nF, nS = hit_pos.numel(), N_row.numel(), L_row.numel(), F_pos.numel(), S_pos.numel()
    fullN = torch.empty(nN, 3, D, device=dev) if nN else None
    fullL = torch.empty(nL, 3, D, device=dev) if nL else None
    for name, t, dt in (('hit_pos', hit_pos, torch.int64), ('hit_slot', hit_slot, torch.int64), ('N_pos', N_pos, torch.int64),
                        ('N_row', N_row, torch.int64), ('L_pos', L_pos, torch.int64), ('L_row', L_row, torch.int64),
                        ('L_off', L_off, torch.int64), ('L_steps', L_steps, torch.int32), ('L_cnt', L_cnt, torch.int32),
                        ('F_pos', F_pos, torch.int64), ('S_pos', S_pos, torch.int64), ('logs', logs, torch.float32),
                        ('ff', ff, torch.float32), ('sw', sw, torch.float32), ('pool', pool, torch.float32)):
        if t.numel() and (t.dtype != dt or not t.is_contiguous() or t.device != dev):
            raise RuntimeError(f'{name} must be a contiguous {dt} tensor on the device of pool')
    if hit_slot.numel() != nh or N_pos.numel() != nN or L_pos.numel() != nL or (nL and (L_steps.numel() != nL * K or L_cnt.numel() != nL)):
        raise RuntimeError('positions and sources of a group must have the same length')
    p = lambda t: t.data_ptr() if t is not None and t.numel() else 0
    with torch.cuda.device(dev):
        st = _lib.lib().srm2_assemble_f32(W.data_ptr(), n, D, p(pool), p(hit_pos), p(hit_slot), nh, p(fullN), p(N_pos), p(N_row), nN,
                                          _seed32(seed), float(bound), p(fullL), p(L_pos), p(L_row), p(logs), p(L_off), p(L_steps),
                                          p(L_cnt), nL, K, table.t.data_ptr(), table.t.shape[0], p(ff), p(F_pos), nF, p(sw), p(S_pos), nS,
                                          _lib.stream_of(dev))
    if st == _lib.SRM2_ERR_UNSUPPORTED and allow_separate_calls:      # odd D / K > 8 / unaligned views: the same result from the separate kernels
        if nh: W.index_copy_(0, hit_pos, pool[:, 0].index_select(0, hit_slot))
        if nN: init_rows(N_row, D, seed, bound, out=fullN); W.index_copy_(0, N_pos, fullN[:, 0])
        if nL: replay_rows(L_row, logs, L_off, L_steps, L_cnt, D, K, seed, bound, table, out=fullL); W.index_copy_(0, L_pos, fullL[:, 0])
        if nF: W.index_copy_(0, F_pos, ff[:, 0])
        if nS: W.index_copy_(0, S_pos, sw)
        return (W, fullN, fullL) if inv is None else (W, fullN, fullL, gather_rows(W, inv, out=emb_out))
    _lib.check(st, 'assemble')
    if inv is None:
        return W, fullN, fullL
    return W, fullN, fullL, gather_rows(W, inv, out=emb_out)


def gather_rows(W, inv, out=None):
    """out[p] = W[inv[p]]: `torch.index_select(W, 0, inv)` of the training step (reference: srm2/train.py:427)."""
    if not W.is_cuda:
        raise RuntimeError('W must be a CUDA tensor: this library has no CPU path')
    n, D = inv.numel(), W.shape[1]
    if out is None:
        out = torch.empty(n, D, device=W.device)
    if inv.dtype != torch.int64 or W.dtype != torch.float32 or not (W.is_contiguous() and inv.is_contiguous() and out.is_contiguous()) or out.numel() != n * D:
        raise RuntimeError('W float32 [rows, D], inv int64 [n] and out float32 [n, D] must be contiguous')
    with torch.cuda.device(W.device):
        st = _lib.lib().srm2_gather_rows_f32(out.data_ptr(), W.data_ptr(), inv.data_ptr(), n, W.shape[0], D, _lib.stream_of(W.device))
    _lib.check(st, 'gather_rows')
    return out
