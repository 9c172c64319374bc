"""Builds libcaminus_b200.so (the CUDA kernels and their C ABI) for sm_100a with nvcc, in-tree.

    python -m caminus_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Flags that matter for parity: -fmad=false (no product and sum is contracted; the kernels
write every fma explicitly), IEEE division and square root, no flush-to-zero, no fast math.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = sorted(glob.glob(os.path.join(HERE, 'csrc', '*.cu')))
HDR = sorted(glob.glob(os.path.join(HERE, 'csrc', '*.cuh')))
OUT = os.path.join(HERE, 'lib', 'libcaminus_b200.so')
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '-lineinfo', '-fmad=false', '-prec-div=true',
         '-prec-sqrt=true', '-ftz=false', '-Xcompiler', '-fPIC', '-shared', '-cudart', 'shared']


def stale():
    if not os.path.isfile(OUT): return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(f) > t for f in SRC + HDR + [os.path.abspath(__file__)])


def build(force=False, verbose=False):
    if not force and not stale(): return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [NVCC] + FLAGS + (['-Xptxas', '-v'] if verbose else []) + ['-o', OUT] + SRC
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode: sys.stderr.write(r.stdout + r.stderr)
    if r.returncode: raise RuntimeError('nvcc failed building libcaminus_b200.so')
    return OUT


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='--verbose' in sys.argv))
