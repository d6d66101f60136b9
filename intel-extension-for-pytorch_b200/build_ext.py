"""Build the PyTorch operator-registration extension (csrc/torch_ext.cpp) in-tree.

    python intel-extension-for-pytorch_b200/build_ext.py [--force]

Produces ipex_b200/_woq_ext.so, linked against ipex_b200/libwoq_b200.so (rpath $ORIGIN).  The
extension holds no kernels: it registers torch_ipex / ipex_prepack operators for the CUDA
dispatch key and forwards to the C ABI."""
import argparse
import hashlib
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "torch_ext.cpp")
OUT_DIR = os.path.join(HERE, "ipex_b200")
OUT = os.path.join(OUT_DIR, "_woq_ext.so")
STAMP = OUT + ".stamp"
BUILD_DIR = os.path.join(HERE, "build", "torch_ext")


def _digest():
    import torch

    h = hashlib.sha256()
    for p in (SRC, os.path.join(HERE, "..", "include", "woq_b200.h")):
        h.update(open(p, "rb").read())
    h.update(torch.__version__.encode())
    return h.hexdigest()


def build(force=False):
    spec = importlib.util.spec_from_file_location("build_native", os.path.join(HERE, "build_native.py"))
    bn = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bn)
    bn.build()
    digest = _digest()
    if not force and os.path.exists(OUT) and os.path.exists(STAMP) and open(STAMP).read().strip() == digest:
        return OUT
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    import ctypes

    ctypes.CDLL(os.path.join(OUT_DIR, "libwoq_b200.so"), mode=ctypes.RTLD_GLOBAL)  # for load()'s dlopen
    built = os.path.join(BUILD_DIR, "woq_b200_torch_ext.so")
    try:
        _load(cpp_extension)
    except OSError:
        # compiled and linked; load() could not dlopen it from the build directory because
        # libwoq_b200.so sits next to the final location, not there
        if not os.path.exists(built):
            raise
    shutil.copyfile(built, OUT + ".new")
    os.replace(OUT + ".new", OUT)  # never rewrite a library that a running process may have mapped
    open(STAMP, "w").write(digest)
    return OUT


def _load(cpp_extension):
    cpp_extension.load(
        name="woq_b200_torch_ext",
        sources=[SRC],
        extra_cflags=["-O2", "-std=c++17"],
        extra_include_paths=[os.path.join(cpp_extension.CUDA_HOME or "/usr/local/cuda", "include")],
        extra_ldflags=[f"-L{OUT_DIR}", "-lwoq_b200", "-Wl,-rpath,'$$ORIGIN'",
                       f"-L{os.path.join(cpp_extension.CUDA_HOME or '/usr/local/cuda', 'lib64')}", "-lcudart",
                       "-lc10_cuda", "-ltorch_cuda"],
        build_directory=BUILD_DIR,
        is_python_module=False,
        with_cuda=True,
        verbose=False,
    )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    print(build(ap.parse_args().force))
