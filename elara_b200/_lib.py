"""ctypes binding of libsrm2_b200.so (the C ABI declared in include/srm2_b200.h).

There is no fallback: if the library is missing or a symbol is absent, importing the bound function
raises, and every non-zero status from the library becomes a RuntimeError.
"""
import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / 'libsrm2_b200.so'

_vp, _i64, _i32, _u32, _f32, _f64, _sz = C.c_void_p, C.c_int64, C.c_int, C.c_uint32, C.c_float, C.c_double, C.c_size_t
_f8 = C.POINTER(C.c_float)

# name -> (restype, argtypes); must list every symbol of include/srm2_b200.h
SIGNATURES = {
    'srm2_version': (C.c_int, []),
    'srm2_status_string': (C.c_char_p, [C.c_int]),
    'srm2_last_cuda_error': (C.c_char_p, []),
    'srm2_launch_count': (C.c_int64, []),
    'srm2_stage_events': (C.c_int, [_vp, _vp]),
    'srm2_verify_exact': (C.c_int, [_i32, C.c_uint64, C.c_uint64, _i32, _i32, _vp, _vp]),
    'srm2_adam_scalars': (C.c_int, [_f64, _f64, _f64, _f64, _i64, _f8]),
    'srm2_adam_rows_f32': (C.c_int, [_vp, _vp, _i32, _vp, _i64, _i64, _f8, _vp]),
    'srm2_init_rows_f32': (C.c_int, [_vp, _vp, _i64, _i64, _u32, _f32, _vp]),
    'srm2_replay_rows_f32': (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _u32, _f32, _vp, _i64, _vp]),
    'srm2_unique_scratch_bytes': (_sz, [_i64]),
    'srm2_unique_inverse_i64': (C.c_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    'srm2_segment_scratch_bytes': (_sz, [_i64, _i64, _i64]),
    'srm2_segment_reduce_f32': (C.c_int, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp, _sz, _vp]),
    'srm2_reduce_adam_f32': (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _i32, _f8, _vp, _sz, _vp]),
    'srm2_route_scratch_bytes': (_sz, [_i64, _i64]),
    'srm2_route_by_owner': (C.c_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    'srm2_dir_scratch_bytes': (_sz, [_i64]),
    'srm2_dir_a': (C.c_int, [_vp, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _i64] + [_vp] * 9 + [_vp, _sz, _vp]),
    'srm2_dir_admit': (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _sz, _vp]),
    'srm2_dir_b': (C.c_int, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _sz, _vp]),
    'srm2_dir_status': (C.c_int, [_vp, _vp, _vp]),
    'srm2_unique_noalloc_max_rows': (C.c_int64, []),
    'srm2_unique_inverse_noalloc_i64': (C.c_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp]),
    'srm2_route_plan': (C.c_int, [_vp, _i64, _i64, _vp, _vp, _sz, _vp]),
    'srm2_route_publish': (C.c_int, [_vp, _vp, _i64, _i64, _vp]),
    'srm2_route_dispatch': (C.c_int, [_vp, _vp, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _i32, _vp, _sz, _vp]),
    'srm2_unique_inverse_nd_i64': (C.c_int, [_vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    'srm2_reduce_adam_nd_f32': (C.c_int, [_vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _i32, _f8, _vp, _sz, _vp]),
    'srm2_reduce_adam_index': (C.c_int, [_vp, _vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _i32, _vp, _sz, _vp]),
    'srm2_reduce_adam_apply_f32': (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _f8, _vp, _sz, _vp]),
    'srm2_reduce_adam_apply_pull_f32': (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _f8, _vp, _sz, _vp]),
    'srm2_presum_request': (C.c_int, [_i64, _vp, _i64, _i64, _vp, _sz, _vp, _vp]),
    'srm2_presum_rows_f32': (C.c_int, [_vp, _i64, _i64, _vp, _vp]),
    'srm2_peer_barrier': (C.c_int, [_vp, _i64, _i64, C.c_uint64, _vp, _i64, _vp, _vp]),
    'srm2_arena_gather_f32': (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    'srm2_arena_scatter_f32': (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    'srm2_gather_rows_f32': (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    'srm2_executor_update_f32': (C.c_int, [_vp, _vp]),
    'srm2_assemble_f32': (C.c_int, [_vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, C.c_uint32, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                    _i64, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _vp]),
    'srm2_plan_scratch_bytes': (_sz, [_i64]),
    'srm2_plan_classify': (C.c_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp,
                                     _vp, _vp, _vp, _vp, _sz, _vp]),
    'srm2_plan_evict_candidates': (C.c_int, [_vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i32, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    'srm2_plan_pack_scratch_bytes': (_sz, [_i64, _i64]),
    'srm2_plan_pack': (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp,
                                 _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    'srm2_staged_steps': (C.c_int, [_vp]),
    'srm2_read_probe': (C.c_int, [_vp, _sz, _vp, _vp]),
    'srm2_route_dispatch_ids': (C.c_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _vp, C.c_uint64, _i64, _vp, _sz, _vp]),
    'srm2_route_publish_barrier': (C.c_int, [_vp, _vp, _vp, _i64, _i64, C.c_uint64, _vp, _i64, _vp]),
    'srm2_route_plan_publish': (C.c_int, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, C.c_uint64, _vp, _i64, _vp, _sz, _vp]),
    'srm2_reduce_adam_pull_f32': (C.c_int, [_vp, _vp, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _i64, _vp, _i64, _f8, _vp, _sz, _vp]),
}



class Staged(C.Structure):
    """srm2_staged of include/srm2_b200.h (every member 8 bytes wide)."""
    _fields_ = ([(k, C.c_int64) for k in ('K', 'first_step', 'n', 'D', 'n_rows', 'cap_u')] +
                [(k, C.c_double) for k in ('lr', 'b1', 'b2', 'eps')] +
                [(k, C.c_void_p) for k in ('pool', 'counts_out', 'ids', 'grads', 'n_k')] +
                [('u', C.c_void_p * 4), ('inv', C.c_void_p * 4), ('scr_s', C.c_void_p * 4)] +
                [('scr_s_bytes', C.c_int64), ('scr_u', C.c_void_p), ('scr_u_bytes', C.c_int64)] +
                [(k, C.c_void_p) for k in ('streams', 'events', 'stage_events', 'trace_events')] +
                [(k, C.c_int64) for k in ('world', 'rank', 'cap', 'n_recv_bufs', 'n_slots', 'timeout_ns')] +
                [('route_scr', C.c_void_p), ('route_scr_bytes', C.c_int64), ('counts', C.c_void_p), ('err', C.c_void_p), ('n_recv', C.c_void_p)] +
                [(k, C.c_void_p) for k in ('cmat', 'recv_lid', 'recv_src', 'peer_cmat', 'peer_lid', 'peer_src', 'slot', 'peer_slot',
                                           'peer_tickets', 'ticket')] +
                [('presum_cap', C.c_int64)] +
                [(k, C.c_void_p) for k in ('peer_req', 'peer_req_n', 'req', 'req_n', 'req_count', 'peer_push', 'peer_out', 'peer_tickets_req',
                                           'peer_tickets_sum', 'presum_done')])


class Presum(C.Structure):
    """srm2_presum of include/srm2_b200.h (every member 8 bytes wide)."""
    _fields_ = ([(k, C.c_int64) for k in ('world', 'rank', 'cap', 'timeout_ns')] + [('err', C.c_void_p), ('peer_tickets', C.c_void_p)] +
                [('ticket', C.c_uint64)] +
                [(k, C.c_void_p) for k in ('peer_req', 'peer_req_n', 'req_count', 'req', 'req_n', 'peer_out', 'done')])


class Update(C.Structure):
    """srm2_update of include/srm2_b200.h."""
    _fields_ = ([(k, C.c_int64) for k in ('D', 'K', 'evl')] + [(k, C.c_void_p) for k in ('G', 'pool', 'glog')] + [('sc', C.c_float * 8)] +
                [(k, C.c_void_p) for k in ('hit_pos', 'hit_slot', 'hrec_dyn', 'hrec_j')] + [('n_hit', C.c_int64)] +
                [('S_pos', C.c_void_p), ('n_S', C.c_int64)] +
                [('fullN', C.c_void_p), ('N_pos', C.c_void_p), ('nNa', C.c_int64), ('nNp', C.c_int64), ('nNc', C.c_int64)] +
                [('fullL', C.c_void_p), ('L_pos', C.c_void_p), ('nLa', C.c_int64), ('nLp', C.c_int64), ('nLc', C.c_int64)] +
                [('ff', C.c_void_p), ('F_pos', C.c_void_p), ('nFa', C.c_int64), ('nFn', C.c_int64)] +
                [('evM_slot', C.c_void_p), ('n_evM', C.c_int64), ('evl_src', C.c_void_p), ('n_evl', C.c_int64)] +
                [(k, C.c_void_p) for k in ('N_adm_slot', 'L_adm_slot', 'F_adm_slot', 'adm_rec_dyn', 'og', 'of', 'oe')])


_lib = None


def lib():
    """The loaded library; raises if it has not been built (python -m elara_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f'{LIB_PATH} is missing: build it with `python -m elara_b200.build` '
                               '(there is no CPU or PyTorch fallback for these kernels)')
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            f = getattr(L, name)          # AttributeError if the symbol is not exported
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


SRM2_ERR_UNSUPPORTED = -2


def check(status, what):
    if status != 0:
        L = lib()
        msg = L.srm2_status_string(status).decode()
        if status == -4:
            msg += ': ' + L.srm2_last_cuda_error().decode()
        raise RuntimeError(f'{what}: {msg} (status {status})')


def ptr(t):
    """Device (or host) address of a tensor's first element; 0 for None."""
    return 0 if t is None else t.data_ptr()


def stream_of(device):
    import torch
    return torch.cuda.current_stream(device).cuda_stream
