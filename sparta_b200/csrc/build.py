"""Build ``libsparta_b200.so`` (the C-ABI library of ``include/sparta_b200.h``) for sm_100a.

Usage: ``python -m sparta_b200.csrc.build [--force] [--verbose]``.  Objects go to ``build/`` at the
repository root, the shared library next to the Python package (``sparta_b200/lib``) so that a
snapshot of the tree carries it.  nvcc cross-compiles without a GPU.
"""
import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
ROOT = os.path.dirname(PKG)
OBJ_DIR = os.path.join(ROOT, 'build', 'obj')
LIB_DIR = os.path.join(PKG, 'lib')
LIB_PATH = os.path.join(LIB_DIR, 'libsparta_b200.so')

NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-lineinfo', '-O3', '-std=c++17',
    '-Xcompiler', '-fPIC',
    '--expt-relaxed-constexpr',
]


def _nvcc() -> str:
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(nvcc):
        raise RuntimeError('nvcc not found: the sm_100a kernels cannot be built')
    return nvcc


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith('.cu'))


def _headers_mtime() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.cuh', '.h'))]
    deps.append(os.path.join(ROOT, 'include', 'sparta_b200.h'))
    return max(os.path.getmtime(d) for d in deps)


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, src[:-3] + '.o')
    path = os.path.join(CSRC, src)
    if not force and os.path.exists(obj):
        if os.path.getmtime(obj) >= max(os.path.getmtime(path), _headers_mtime()):
            return obj
    cmd = [_nvcc(), *NVCC_FLAGS, '-c', path, '-o', obj]
    if verbose:
        cmd.insert(1, '-Xptxas')
        cmd.insert(2, '-v')
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(f'$ {" ".join(cmd)}\n{res.stdout}{res.stderr}')
    if res.returncode != 0:
        raise RuntimeError(f'nvcc failed on {src}')
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of this directory and link the shared library; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    srcs = _sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < newest:
        cmd = [_nvcc(), '-shared', '-o', LIB_PATH, *objs, '-gencode', 'arch=compute_100a,code=sm_100a',
               '-Xcompiler', '-fPIC']
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError('linking libsparta_b200.so failed')
    return LIB_PATH


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(a.force, a.verbose))
