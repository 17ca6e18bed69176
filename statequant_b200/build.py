"""Builds the CUDA extension in-tree: ``statequant_b200/lib/libstatequant_b200.so`` (sm_100a only).

    python -m statequant_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  ``--fmad=false`` stops the compiler from contracting separately rounded
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
UNITS = ['sqb200.cu']


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
    cmd = [_nvcc(), '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-lineinfo', '-std=c++17',
           '--fmad=false', '-Xcompiler', '-fPIC', '-shared', '-cudart', 'static',
           '-o', OUT] + [os.path.join(SRC, u) for u in UNITS]
    cmd += os.environ.get('SQB_NVCC_EXTRA', '').split()
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError('nvcc failed:\n' + ' '.join(cmd) + '\n' + r.stdout + r.stderr)
    if verbose:
        print(r.stdout + r.stderr)
    return OUT


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
