"""Builds the CUDA library of this package in-tree with nvcc for sm_100a.

    python -m hgq2_b200.build            # build if sources are newer than the library
    python -m hgq2_b200.build --force

The output is hgq2_b200/lib/libhgq_b200.so, a plain C-ABI shared library (no torch or Python
headers) that hgq2_b200._lib loads with ctypes.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / 'csrc'
LIBDIR = PKG / 'lib'
OBJDIR = LIBDIR / 'obj'
LIB = LIBDIR / 'libhgq_b200.so'

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-O3', '-lineinfo', '-std=c++17',
    '-Xcompiler', '-fPIC',
    '-Xptxas', '-v',
]


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError('nvcc not found')


def sources() -> list[Path]:
    return sorted(CSRC.glob('*.cu'))


def _deps_mtime() -> float:
    files = list(CSRC.glob('*.cu')) + list(CSRC.glob('*.cuh')) + list((PKG.parent / 'include').glob('*.h'))
    return max(f.stat().st_mtime for f in files)


def needs_build() -> bool:
    return not LIB.exists() or LIB.stat().st_mtime < _deps_mtime()


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    OBJDIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    dep_m = _deps_mtime()

    def compile_one(src: Path) -> Path:
        obj = OBJDIR / (src.stem + '.o')
        if not force and obj.exists() and obj.stat().st_mtime >= dep_m:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, '-c', str(src), '-o', str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OBJDIR / (src.stem + '.ptxas.log')).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f'nvcc failed for {src.name}:\n{r.stderr[-4000:]}')
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [nvcc, '-shared', '-o', str(LIB), *map(str, objs), '-lcudart']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'link failed:\n{r.stderr[-4000:]}')
    return LIB


if __name__ == '__main__':
    path = build(force='--force' in sys.argv, verbose='-v' in sys.argv)
    print(path)
