"""Compile the reference's own C++ sources for this path into oracle/_ref/ (test infrastructure).

The two translation units are compiled where they lie in the reference checkout; no reference source
is copied.  The outputs are ordinary CPython extension modules (pybind11 + libtorch, both part of
the image), loadable with importlib on any machine that has the same image:

  oracle/_ref/srm2_cpu_ext_<level>.so   <- srm2/csrc/srm2_cpu.cpp   (cpu_adam, adam_scalars, ...)
  oracle/_ref/srm2_elara_dir.so         <- srm2/csrc/elara_dir.cpp  (elara_dir_a, elara_dir_b)
  oracle/_ref/srm2/*.py                 <- srm2/*.py, staged unchanged so that the reference's own planner, executor and
                                           Triton kernels can be run on the GPU box beside this library (the tests that
                                           need them skip when the folder is absent).  oracle/_ref/ is never tracked and
                                           nothing under elara_b200/ imports it.

The reference builds srm2_cpu.cpp with `-O3 -ffp-contract=off -march=native -fno-fast-math`
(srm2/ops.py:23-25).  `-march=native` cannot travel between machines, so two fixed ISA levels are
built instead (x86-64-v3 = AVX2, x86-64-v4 = AVX-512) and the loader picks the highest one the host
CPU supports; contraction stays off, so the results are the same bits at either level.
elara_dir.cpp uses the reference's `-O2` (srm2/ops.py:37).

Usage: python oracle/build_ref.py --ref /path/to/reference      (or SRM2_REFERENCE=/path/to/reference)
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / '_ref'


def _flags():
    import pybind11
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f'-I{p}' for p in ce.include_paths()] + [f'-I{pybind11.get_include()}', f'-I{sysconfig.get_paths()["include"]}']
    libdir = ce.library_paths()[0]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ['-std=c++17', '-fPIC', '-shared', f'-D_GLIBCXX_USE_CXX11_ABI={abi}', '-DTORCH_API_INCLUDE_EXTENSION_H',
              '-w'] + inc
    link = [f'-L{libdir}', f'-Wl,-rpath,{libdir}', '-ltorch', '-ltorch_cpu', '-lc10', '-ltorch_python', '-lpthread']
    return common, link


def stage_python(ref):
    """Copies the reference's Python package into the (untracked) oracle/_ref/srm2 for the tests that run it."""
    import shutil
    src = Path(ref) / 'srm2'
    dst = OUT / 'srm2'
    dst.mkdir(parents=True, exist_ok=True)
    for f in sorted(src.glob('*.py')):
        shutil.copyfile(f, dst / f.name)
    return dst


def build(ref=None, force=False):
    ref = ref or os.environ.get('SRM2_REFERENCE')
    if not ref:
        return False
    ref = Path(ref)
    src_cpu = ref / 'srm2/csrc/srm2_cpu.cpp'
    src_dir = ref / 'srm2/csrc/elara_dir.cpp'
    if not src_cpu.exists():
        return False
    OUT.mkdir(exist_ok=True)
    stage_python(ref)
    common, link = _flags()
    jobs = []
    for level in ('x86-64-v3', 'x86-64-v4'):
        name = 'srm2_cpu_ext_' + level.split('-')[-1]
        jobs.append((src_cpu, OUT / f'{name}.so', name,
                     ['-O3', '-ffp-contract=off', f'-march={level}', '-fno-fast-math']))
    jobs.append((src_dir, OUT / 'srm2_elara_dir.so', 'srm2_elara_dir', ['-O2']))
    procs = []
    for src, out, name, opt in jobs:
        if out.exists() and not force and out.stat().st_mtime >= src.stat().st_mtime:
            continue
        cmd = ['g++', *opt, *common, f'-DTORCH_EXTENSION_NAME={name}', str(src), '-o', str(out), *link]
        procs.append((out, subprocess.Popen(cmd)))
    ok = True
    for out, p in procs:
        if p.wait() != 0:
            ok = False
            print(f'build_ref: failed to build {out}', file=sys.stderr)
    return ok


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref', default=os.environ.get('SRM2_REFERENCE'), help='the reference checkout (or set SRM2_REFERENCE)')
    ap.add_argument('--force', action='store_true')
    a = ap.parse_args()
    sys.exit(0 if build(a.ref, a.force) else 1)
