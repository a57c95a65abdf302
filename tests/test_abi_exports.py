"""The C-ABI library loads and exports every symbol that include/*.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    syms = set()
    for h in (ROOT / 'include').glob('*.h'):
        text = re.sub(r'/\*.*?\*/', '', h.read_text(), flags=re.S)
        syms |= set(re.findall(r'\b(srm2_[a-z0-9_]+)\s*\(', text))
    return syms


def test_library_exports_every_declared_symbol():
    from elara_b200 import build, _lib
    so = build.build()
    L = ctypes.CDLL(str(so))
    syms = declared_symbols()
    assert len(syms) >= 7
    for s in syms:
        assert hasattr(L, s), f'{s} is declared in include/ but not exported'
    # the Python binding lists exactly the declared symbols
    assert set(_lib.SIGNATURES) == syms


def test_host_entry_points_without_gpu(oracle):
    import numpy as np
    from elara_b200 import ops, _lib
    L = _lib.lib()
    assert L.srm2_version() >= 100
    assert L.srm2_status_string(0) == b'ok' and L.srm2_status_string(-3) == b'scratch buffer too small'
    for step in (1, 2, 17, 100, 12345):
        got = np.array(ops.ext().adam_scalars(1e-3, 0.9, 0.999, 1e-8, step), np.float32)
        assert np.array_equal(got.view(np.uint32), oracle.adam_scalars(1e-3, 0.9, 0.999, 1e-8, step).view(np.uint32))


def test_no_cpu_path():
    import pytest
    import torch
    from elara_b200 import ops, gpu_ops
    with pytest.raises(RuntimeError):
        ops.gpu_adam(torch.zeros(4, 3, 8), torch.arange(2), torch.zeros(2, 8), 1e-3, .9, .999, 1e-8, 1)
    with pytest.raises(RuntimeError):
        gpu_ops.init_rows(torch.arange(3), 8, 1, 0.01)
    with pytest.raises(AttributeError):
        ops.ext().cpu_adam


def test_struct_layouts_match_the_header(tmp_path):
    """The ctypes mirrors of the header's structs have the size and member offsets a C compiler gives them."""
    import subprocess
    from elara_b200 import _lib
    src = tmp_path / 'layout.c'
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "srm2_b200.h"\n'
                   'int main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(srm2_staged), offsetof(srm2_staged, pool), offsetof(srm2_staged, u),\n'
                   '                        offsetof(srm2_staged, world), offsetof(srm2_staged, ticket));\n'
                   '  printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(srm2_update), offsetof(srm2_update, sc), offsetof(srm2_update, hit_pos),\n'
                   '         offsetof(srm2_update, nNa), offsetof(srm2_update, evl_src), offsetof(srm2_update, oe)); return 0; }\n')
    exe = tmp_path / 'layout'
    subprocess.check_call(['gcc', '-I', str(ROOT / 'include'), '-o', str(exe), str(src)])
    lines = subprocess.check_output([str(exe)]).decode().splitlines()
    size, o_pool, o_u, o_world, o_ticket = map(int, lines[0].split())
    S = _lib.Staged
    assert (ctypes.sizeof(S), S.pool.offset, S.u.offset, S.world.offset, S.ticket.offset) == (size, o_pool, o_u, o_world, o_ticket)
    U = _lib.Update
    assert (ctypes.sizeof(U), U.sc.offset, U.hit_pos.offset, U.nNa.offset, U.evl_src.offset, U.oe.offset) == tuple(map(int, lines[1].split()))
