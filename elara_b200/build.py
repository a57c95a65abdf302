"""Build recipe of libsrm2_b200.so: nvcc, sm_100a only, no torch headers.

    python -m elara_b200.build [--force] [--verbose]

The library is built in-tree (elara_b200/libsrm2_b200.so).  -fmad=false keeps every fp32 multiply and add
a separately rounded operation (the kernels also use the __f*_rn intrinsics, which are never contracted);
division and square root are the IEEE-rounded forms (-prec-div/-prec-sqrt are nvcc's defaults and are stated
explicitly); subnormals are kept (-ftz=false).
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / 'csrc'
OBJ = CSRC / 'build'
LIB = PKG / 'libsrm2_b200.so'

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '-fmad=false', '-ftz=false',
              '-prec-div=true', '-prec-sqrt=true', '-Xcompiler', '-fPIC', f'-I{ROOT / "include"}', f'-I{CSRC}']


def sources():
    return sorted(CSRC.glob('*.cu'))


def _nvcc():
    for c in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if c and (os.path.sep not in c or os.path.exists(c)):
            return c
    return 'nvcc'


def up_to_date():
    if not LIB.exists():
        return False
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh')) + list((ROOT / 'include').glob('*.h'))
    return all(d.stat().st_mtime <= t for d in deps)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    extra = ['-Xptxas', '-v'] if verbose else []

    def cc(src):
        obj = OBJ / (src.stem + '.o')
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, '-c', str(src), '-o', str(obj)], capture_output=True, text=True)
        return src, obj, r

    with ThreadPoolExecutor(max_workers=8) as ex:
        res = list(ex.map(cc, sources()))
    for src, obj, r in res:
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f'nvcc failed on {src.name}')
    objs = [str(o) for _, o, _ in res]
    subprocess.check_call([nvcc, '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', str(LIB), *objs, '-lcudart'])
    return LIB


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(a.force, a.verbose))
