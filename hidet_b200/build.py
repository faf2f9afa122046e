"""Builds ``libhidet_b200q.so`` in-tree from ``hidet_b200/csrc`` with nvcc for sm_100a.

The library is prebuilt and loaded with ctypes, the way the reference loads its own compiled
libraries (python/hidet/ffi/ffi.py:32-69); nothing is compiled at import time.

Run ``python -m hidet_b200.build`` (add ``--force`` to rebuild everything, ``--verbose`` for
ptxas resource usage).
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, 'csrc')
OBJ_DIR = os.path.join(PKG_DIR, 'csrc', 'build')
LIB_DIR = os.path.join(PKG_DIR, 'lib')
LIB_NAME = 'libhidet_b200q.so'
LIB_PATH = os.path.join(LIB_DIR, LIB_NAME)

ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a']
COMMON_FLAGS = ['-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden']

# Flags that differ per translation unit.  The quantize kernels are compiled with the two
# floating-point flags the reference compiles its generated kernels with
# (python/hidet/backend/build.py:164-177), because they decide how an f32 division is evaluated.
PER_SOURCE_FLAGS: Dict[str, List[str]] = {'quantize.cu': ['-ftz=true', '-prec-div=false']}


def find_nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found: set NVCC or put it on PATH')


def sources() -> List[str]:
    return sorted(f for f in os.listdir(SRC_DIR) if f.endswith('.cu'))


def _newest_header_mtime() -> float:
    mt = 0.0
    for root in (SRC_DIR, os.path.join(PKG_DIR, '..', 'include')):
        for f in os.listdir(root):
            if f.endswith(('.h', '.cuh')):
                mt = max(mt, os.path.getmtime(os.path.join(root, f)))
    return mt


def _compile(nvcc: str, src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, src[:-3] + '.o')
    cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *PER_SOURCE_FLAGS.get(src, []), '-c', os.path.join(SRC_DIR, src), '-o', obj]
    if verbose:
        cmd[1:1] = ['-Xptxas', '-v']
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError('nvcc failed for {}:\n{}\n{}'.format(src, ' '.join(cmd), res.stdout))
    if verbose and res.stdout:
        print(res.stdout)
    return obj


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile what is out of date and link the shared library.  Returns its path."""
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    stale = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + '.o')
        src_mtime = max(os.path.getmtime(os.path.join(SRC_DIR, src)), hdr_mtime, os.path.getmtime(__file__))
        if force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < src_mtime:
            stale.append(src)
    if stale:
        with ThreadPoolExecutor(max_workers=min(8, len(stale))) as pool:
            list(pool.map(lambda s: _compile(nvcc, s, verbose), stale))
    objs = [os.path.join(OBJ_DIR, s[:-3] + '.o') for s in sources()]
    if stale or not os.path.exists(LIB_PATH):
        cmd = [nvcc, *ARCH_FLAGS, '-shared', '-o', LIB_PATH, *objs, '-cudart', 'static']
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError('link failed:\n{}\n{}'.format(' '.join(cmd), res.stdout))
    return LIB_PATH


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true', help='print ptxas resource usage (forces a recompile)')
    args = ap.parse_args(argv)
    print(build_library(force=args.force, verbose=args.verbose))
    return 0


if __name__ == '__main__':
    sys.exit(main())
