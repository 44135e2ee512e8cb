"""Builds n2d2_b200/libn2d2b.so (CUDA kernels + C ABI) for sm_100a with nvcc, in-tree."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
OUT = os.path.join(HERE, 'libn2d2b.so')
SOURCES = ['net.cu', 'simt_kernels.cu', 'igemm_tcgen05.cu', 'stem_tcgen05.cu', 'patch_tcgen05.cu', 'stem_s2d_tcgen05.cu',
           'probe_tcgen05.cu']
HEADERS = ['common.cuh', 'kernels.h', 'tc_common.cuh', 'host_internal.h', os.path.join('..', '..', 'include', 'n2d2b.h')]
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-shared', '-diag-suppress', '550']


def _nvcc():
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return 'nvcc'


def needs_build():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """One nvcc process per source file (in parallel), objects under n2d2_b200/_build/, then one link step whose
    output replaces the library atomically."""
    if not force and not needs_build():
        return OUT
    from concurrent.futures import ThreadPoolExecutor
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a compiler wrapper without its support files
    env.pop('CC', None)
    env.pop('CXX', None)
    objdir = os.path.join(HERE, '_build')
    os.makedirs(objdir, exist_ok=True)
    newest_header = max(os.path.getmtime(os.path.join(CSRC, h)) for h in HEADERS)
    flags = [f for f in NVCC_FLAGS if f != '-shared'] + (['-Xptxas', '-v'] if verbose else [])

    def compile_one(src):
        obj = os.path.join(objdir, os.path.splitext(src)[0] + '.o')
        path = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), newest_header):
            return obj
        subprocess.check_call([_nvcc()] + flags + ['-c', path, '-o', obj], env=env)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    tmp = OUT + '.tmp'
    subprocess.check_call([_nvcc(), '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', '-o', tmp] + objs, env=env)
    os.replace(tmp, OUT)
    return OUT


if __name__ == '__main__':
    print(build_library(force='--force' in sys.argv, verbose='-v' in sys.argv))
