"""Build recipe of the native library: one nvcc call, sm_100a only, output in-tree.

    python -m triteia_b200.build

produces triteia_b200/libtriteia_b200.so from triteia_b200/csrc/triteia_b200.cu (a single
translation unit).  nvcc cross-compiles without a GPU.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(PKG, "csrc", "triteia_b200.cu")
LIB = os.path.join(PKG, "libtriteia_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    d = os.path.join(PKG, "csrc")
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cu", ".cuh")))


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    hdr = os.path.join(PKG, "..", "include", "triteia_b200.h")
    return any(os.path.getmtime(p) > t for p in sources() + [hdr])


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [SRC, "-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libtriteia_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
