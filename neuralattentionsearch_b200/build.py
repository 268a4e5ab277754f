"""Builds libnats_b200.so (the C-ABI library with every CUDA kernel) in-tree with nvcc for sm_100a.

    python -m neuralattentionsearch_b200.build [--force]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libnats_b200.so')
SOURCES = ['cache_ops.cu', 'decode.cu', 'prefill_sm100.cu', 'rope.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17',
              '-Xcompiler', '-fPIC', '-Xcompiler', '-fvisibility=hidden', '--use_fast_math']


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found (set NVCC or put it on PATH)')


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, '..', 'include', 'nats_b200.h'), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = _nvcc()
    objs = []
    build_dir = os.path.join(HERE, 'build')
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace('.cu', '.o'))
        cmd = [nvcc, *NVCC_FLAGS, '-c', os.path.join(CSRC, src), '-o', obj]
        if verbose:
            cmd.insert(1, '-Xptxas=-v')
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode:
            sys.stderr.write(out)
        if pr.returncode:
            raise RuntimeError(f'nvcc failed on {src}')
    cmd = [nvcc, '-shared', '-o', LIB, *objs, '-gencode', 'arch=compute_100a,code=sm_100a']
    subprocess.run(cmd, check=True)
    return LIB


WAIT_TEST_LIB = os.path.join(HERE, '..', 'tests', '_build', 'libnats_b200_waittest.so')


def build_wait_test(force: bool = False) -> str:
    """A TEST-ONLY build of the prefill entry points (never loaded by the package): every bounded wait gives up after 3 ms
    instead of 400 ms and the K/V producer withholds one V tile per CTA, so that a test can watch a wait run out, the kernel
    return with a status code and the context stay usable."""
    lib = os.path.abspath(WAIT_TEST_LIB)
    srcs = [os.path.join(CSRC, f) for f in ('prefill_sm100.cu', 'cache_ops.cu')]
    if not force and os.path.exists(lib) and all(os.path.getmtime(x) <= os.path.getmtime(lib) for x in srcs + [__file__]):
        return lib
    os.makedirs(os.path.dirname(lib), exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, '-DNATS_WAIT_LIMIT_NS=3000000ull', '-DNATS_TEST_WITHHOLD_FIRST_V=1', '-shared', '-o', lib, *srcs]
    subprocess.run(cmd, check=True)
    return lib


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv))
