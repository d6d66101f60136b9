"""Loads the operator-registration extension so that torch.ops.torch_ipex.* and
torch.ops.ipex_prepack.* exist.  No fallback: a missing extension is an error."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
EXT_PATH = os.path.join(_HERE, "_woq_ext.so")
_loaded = False


def load_ops():
    global _loaded
    if _loaded:
        return
    from . import _capi

    if not os.path.exists(EXT_PATH):
        raise RuntimeError(
            f"{EXT_PATH} is missing: build it with "
            "`python intel-extension-for-pytorch_b200/build_ext.py` (there is no eager fallback)")
    ctypes.CDLL(_capi.LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(EXT_PATH)
    _loaded = True
