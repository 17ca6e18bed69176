"""Builds the CUDA extension in-tree: ``statequant_b200/lib/libstatequant_b200.so`` (sm_100a only).

    python -m statequant_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU; the translation units compile in parallel and are linked into one library.  ``--fmad=false`` stops the compiler from contracting separately rounded
products into FMAs (every FMA the kernels want is written explicitly), and there is no fast-math flag: the stored
codes depend on IEEE division, square root and round-half-even.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, 'csrc')
OUT_DIR = os.path.join(HERE, 'lib')
OUT = os.path.join(OUT_DIR, 'libstatequant_b200.so')
UNITS = ['sqb200.cu', 'staged_gdn.cu', 'staged_m2.cu', 'staged_kda.cu', 'fold_launch.cu', 'mma_gdn.cu', 'mma_m2.cu',
         'mma_kda.cu', 'gga_reg.cu']


def _nvcc():
    for c in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if c and os.path.exists(c):
            return c
    raise RuntimeError('nvcc not found (set NVCC)')


def sources():
    out = []
    for root, _, files in os.walk(SRC):
        out += [os.path.join(root, f) for f in files if f.endswith(('.cu', '.cuh', '.h'))]
    out.append(os.path.join(HERE, '..', 'include', 'statequant_b200.h'))
    return out


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(s) <= t for s in sources())


def build(force=False, verbose=False):
    """Compile if the library is missing or older than a source file.  Returns the library path."""
    if not force and up_to_date():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(OUT_DIR, 'obj')
    os.makedirs(obj_dir, exist_ok=True)
    flags = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-lineinfo', '-std=c++17', '--fmad=false',
             '-Xcompiler', '-fPIC'] + os.environ.get('SQB_NVCC_EXTRA', '').split()
    if verbose:
        flags += ['-Xptxas', '-v']
    units = os.environ.get('SQB_UNITS', '').split() or UNITS     # a subset recompiles only those objects

    def compile_unit(u):
        obj = os.path.join(obj_dir, u[:-3] + '.o')
        cmd = [_nvcc()] + flags + ['-c', os.path.join(SRC, u), '-o', obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return u, cmd, r

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 1)) as pool:
        for u, cmd, r in pool.map(compile_unit, units):
            if r.returncode != 0:
                raise RuntimeError('nvcc failed:\n' + ' '.join(cmd) + '\n' + r.stdout + r.stderr)
            if verbose:
                print(f'==== {u}\n' + r.stdout + r.stderr)
    objs = [os.path.join(obj_dir, u[:-3] + '.o') for u in UNITS]
    missing = [o for o in objs if not os.path.exists(o)]
    if missing:
        raise RuntimeError('objects missing (build all units first): ' + ' '.join(missing))
    cmd = [_nvcc(), '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', '-cudart', 'static', '-o', OUT] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError('link failed:\n' + ' '.join(cmd) + '\n' + r.stdout + r.stderr)
    return OUT


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
