# -*- coding: utf-8 -*-
"""Build ``libmgwfbp_b200.so`` in-tree with nvcc for sm_100a.

``python -m mgwfbp_b200.ops.build [--verbose] [--force] [--checked]``.  Every ``.cu`` under ``csrc/`` is compiled to
an object (only when stale) and linked into ``mgwfbp_b200/lib/libmgwfbp_b200.so``.  The CUDA runtime
is linked statically, so the library only needs the driver at load time and can be loaded in a
process that also runs PyTorch.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from typing import List

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIR = os.path.join(PKG_DIR, 'csrc')
LIB_DIR = os.path.join(PKG_DIR, 'lib')
OBJ_DIR = os.path.join(LIB_DIR, 'obj')
LIB_PATH = os.path.join(LIB_DIR, 'libmgwfbp_b200.so')
# the same sources with -DMGW_CHECKED: index checks inside the table-driven kernels (csrc/common.cuh)
CHECKED_OBJ_DIR = os.path.join(LIB_DIR, 'obj_checked')
CHECKED_LIB_PATH = os.path.join(LIB_DIR, 'libmgwfbp_b200_checked.so')

ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a']
COMMON = ['-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC', '--expt-relaxed-constexpr']


def nvcc_path() -> str:
    cand = os.environ.get('NVCC') or shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.isfile(cand):
        raise RuntimeError('nvcc not found (set NVCC=/path/to/nvcc)')
    return cand


def sources() -> List[str]:
    return sorted(os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith('.cu'))


def _stale(target: str, deps: List[str]) -> bool:
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False, checked: bool = False) -> str:
    obj_dir, lib_path = (CHECKED_OBJ_DIR, CHECKED_LIB_PATH) if checked else (OBJ_DIR, LIB_PATH)
    extra = ['-DMGW_CHECKED=1'] if checked else []
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = nvcc_path()
    headers = [os.path.join(SRC_DIR, f) for f in os.listdir(SRC_DIR) if f.endswith(('.h', '.cuh'))]
    objs, rebuilt = [], False
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + '.o')
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + ARCH_FLAGS + COMMON + extra + (['-Xptxas', '-v'] if verbose else []) + ['-I', SRC_DIR, '-c', src, '-o', obj]
            if verbose:
                print(' '.join(cmd), flush=True)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError('nvcc failed on %s' % src)
            rebuilt = True
    if rebuilt or force or _stale(lib_path, objs):
        cmd = [nvcc] + ARCH_FLAGS + ['-shared', '-cudart', 'static', '-o', lib_path] + objs
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError('link failed')
    return lib_path


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--verbose', action='store_true')
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--checked', action='store_true', help='build libmgwfbp_b200_checked.so (kernels verify their indices)')
    a = ap.parse_args()
    print(build(a.verbose, a.force, a.checked))
