"""Build ``libmsamp_b200.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m msamp.ops.build [--force] [--verbose]``.
The library has a C ABI and does not link against torch, so it compiles in seconds per file.
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, 'csrc')
OBJ = os.path.join(HERE, 'build')
OUT = os.path.join(HERE, 'libmsamp_b200.so')

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '--use_fast_math',
    '-Xcompiler', '-fPIC', '-Xcompiler', '-Wall', '--expt-relaxed-constexpr', '-I', SRC,
]


def _nvcc():
    exe = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(exe):
        raise RuntimeError('nvcc not found')
    return exe


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    """Compile every ``csrc/*.cu`` and link the shared library. Returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(SRC, '*.cu')))
    headers = glob.glob(os.path.join(SRC, '*.cuh')) + glob.glob(os.path.join(SRC, '*.h'))
    nvcc = _nvcc()
    jobs = []
    objects = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + '.o')
        objects.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-c', src, '-o', obj]
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, res

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for cmd, res in pool.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(' '.join(cmd) + '\n' + res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError(f'nvcc failed for {cmd[-3]}')
    if force or jobs or _stale(OUT, objects):
        cmd = [nvcc, '-shared', '-o', OUT] + objects + ['-lcudart']
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError('link failed')
    return OUT


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
