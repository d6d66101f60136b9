"""Build libwoq_b200.so (CUDA kernels + C ABI) in-tree for sm_100a with nvcc.

    python intel-extension-for-pytorch_b200/build_native.py [--force] [--verbose]

The shared library lands next to the Python package (ipex_b200/libwoq_b200.so) so that it
travels with the source tree; nothing is installed into site-packages.
"""
import argparse
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "ipex_b200")
LIB = os.path.join(OUT_DIR, "libwoq_b200.so")
STAMP = LIB + ".stamp"

CUDA_SOURCES = [
    "woq_capi.cu",
    "woq_pack.cu",
    "woq_decode_int4.cu",
    "woq_int4_tc.cu",
    "woq_int8.cu",
    "woq_static_scratch.cu",
    "woq_generic.cu",
    "woq_int8_block.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xlinker", "-soname=libwoq_b200.so",
]


def _nvcc():
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _digest():
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + ["../../include/woq_b200.h"]
    for n in names:
        p = os.path.join(CSRC, n)
        if os.path.isfile(p) and n.endswith((".cu", ".cuh", ".h")):
            h.update(n.encode())
            h.update(open(p, "rb").read())
    h.update(" ".join(NVCC_FLAGS + os.environ.get("WOQ_NVCC_EXTRA", "").split()).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compile if sources changed; returns the path of the library."""
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(STAMP):
        if open(STAMP).read().strip() == digest:
            return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    extra = os.environ.get("WOQ_NVCC_EXTRA", "").split()
    cmd = [_nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else [])
    # link into a temporary name and rename: a process that has the old library mapped keeps its
    # own copy instead of seeing the file change under it
    tmp = LIB + ".new"
    cmd += [os.path.join(CSRC, s) for s in CUDA_SOURCES] + ["-o", tmp]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libwoq_b200.so")
    os.replace(tmp, LIB)
    open(STAMP, "w").write(digest)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
