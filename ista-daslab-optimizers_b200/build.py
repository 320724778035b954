"""Builds libmicroadam_b200.so (sm_100a) in-tree with nvcc.

    python build.py [--verbose] [--force]

The CUDA runtime is linked statically, so loading the library needs no CUDA libraries; the
first call into it needs an NVIDIA driver.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OUT_DIR = os.path.join(HERE, 'ista_daslab_optimizers_b200', 'lib')
LIB_PATH = os.path.join(OUT_DIR, 'libmicroadam_b200.so')
INCLUDE = os.path.join(os.path.dirname(HERE), 'include')


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found (set NVCC or put it on PATH)')


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith('.cu'))


def _inputs():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return deps


def up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(p) <= t for p in _inputs())


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and up_to_date():
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    obj_dir = os.path.join(HERE, 'build')
    os.makedirs(obj_dir, exist_ok=True)
    common = [_nvcc(), '-O3', '-std=c++17', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo',
              '-Xcompiler', '-fPIC', '-I', INCLUDE]
    if verbose:
        common += ['-Xptxas', '-v']
    if os.environ.get('MAB_STATS'):
        common += ['-DMAB_STATS']       # development-only tile statistics
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + '.o')
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ['-c', src, '-o', obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f'--- {os.path.basename(src)}\n{out}\n')
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError('nvcc failed')
    link = [_nvcc(), '-shared', '-cudart', 'static', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', LIB_PATH] + objs
    subprocess.run(link, check=True)
    return LIB_PATH


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--verbose', action='store_true', help='print ptxas register / shared-memory usage')
    ap.add_argument('--force', action='store_true')
    args = ap.parse_args()
    print(build(verbose=args.verbose, force=args.force))
