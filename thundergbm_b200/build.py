"""Builds libthundergbm.so and the two CLI binaries in-tree for sm_100a with nvcc.

    python -m thundergbm_b200.build [--force]

-fmad=false: no implicit fused multiply-add; the one place where the reference's compiled code
contracts (y_pred += lr * w) is written with an explicit fma, so results do not depend on the
compiler's contraction choices and can be restated exactly on the host.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, 'csrc')
LIB = os.path.join(HERE, 'libthundergbm.so')
BIN = os.path.join(HERE, 'bin')
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
FLAGS = ['-std=c++17', '-O3', '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-fmad=false',
         '-Xcompiler', '-fPIC,-O3', '-ccbin', '/usr/bin/g++']
SOURCES = ['tgbm_booster.cu', 'tgbm_predictor.cu', 'tgbm_capi.cu', 'tgbm_host.cpp', 'tgbm_comm.cpp', 'tgbm_noalloc.cu', 'tgbm_devmem.cu']


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.h', '.cuh'))]
    hdrs.append(os.path.join(HERE, '..', 'include', 'thundergbm.h'))
    objs = []
    os.makedirs(os.path.join(HERE, 'build'), exist_ok=True)
    procs = []
    for s in srcs:
        o = os.path.join(HERE, 'build', os.path.basename(s) + '.o')
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC] + FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-x', 'cu', '-c', s, '-o', o]
            procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stdout.write(out)
        if p.returncode:
            raise RuntimeError(f'nvcc failed on {s}')
    if force or procs or not os.path.exists(LIB):
        # linked beside the target and renamed: whoever copies or loads the tree meanwhile sees a complete library
        subprocess.check_call([NVCC, '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-ccbin', '/usr/bin/g++',
                               '-o', LIB + '.tmp'] + objs + ['-ldl'])
        os.replace(LIB + '.tmp', LIB)
    os.makedirs(BIN, exist_ok=True)
    for name in ('thundergbm_train', 'thundergbm_predict'):
        src = os.path.join(CSRC, 'cli', name + '.cu')
        exe = os.path.join(BIN, name.replace('_', '-'))
        if force or _newer(exe, [src, LIB]):
            subprocess.check_call([NVCC] + FLAGS + [src, '-o', exe + '.tmp', '-L' + HERE, '-lthundergbm',
                                                    '-Xlinker', '-rpath', '-Xlinker', '$ORIGIN/..'])
            os.replace(exe + '.tmp', exe)
    return LIB


if __name__ == '__main__':
    build(force='--force' in sys.argv, verbose='-v' in sys.argv)
    print(LIB)
