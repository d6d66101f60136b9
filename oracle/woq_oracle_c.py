"""ctypes wrapper of oracle/_build/libwoq_oracle.so (the C restatement in woq_oracle_c.c).

TEST INFRASTRUCTURE ONLY: used by tests and by the CPU-baseline leg of the benchmark."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "libwoq_oracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        L.woq_oracle_layer_create.restype = vp
        L.woq_oracle_layer_create.argtypes = [vp, ci, ci, ci, vp, vp, vp, ci, ci]
        L.woq_oracle_layer_free.argtypes = [vp]
        L.woq_oracle_linear_bf16.argtypes = [vp, vp, ci, ci, vp, vp, vp, ci]
        L.woq_oracle_linear_int8.argtypes = [vp, vp, ci, ci, vp, vp, vp, vp, ci]
        L.woq_oracle_linear_fp16_small_m.argtypes = [vp, vp, ci, ci, vp, vp, vp, ci]
        L.woq_oracle_has_fp16_kernel.restype = ci
        L.woq_oracle_quant_act_sym.argtypes = [vp, ci, ci, vp, vp]
        L.woq_oracle_max_threads.restype = ci
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _bf16_bits(x):
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def _from_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


class Layer:
    """One quantised layer packed into the reference's blocked layout."""

    def __init__(self, qweight, n, k, scales, zps, bias, group_size, is_int8=False, int8_compute=False):
        self.n, self.k = n, k
        qw = np.ascontiguousarray(qweight).view(np.uint8)
        s = np.ascontiguousarray(np.asarray(scales, dtype=np.float32).reshape(n, -1))
        z = None if zps is None else np.ascontiguousarray(np.asarray(zps, dtype=np.float32).reshape(n, -1))
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self._h = lib().woq_oracle_layer_create(_p(qw), n, k, int(is_int8), _p(s), _p(z), _p(b),
                                                int(group_size), int(int8_compute))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().woq_oracle_layer_free(self._h)
            self._h = None

    def linear_bf16(self, x, fusion=0, others=(), threads=0):
        """x: float32 array of bf16 values [M,K] -> float32 array of bf16 values."""
        xb = _bf16_bits(x)
        m = xb.shape[0]
        n_out = self.n // 2 if fusion == 0x100 else self.n
        y = np.empty((m, n_out), dtype=np.uint16)
        o = [_bf16_bits(t) for t in others]
        lib().woq_oracle_linear_bf16(self._h, _p(xb), m, fusion, _p(o[0]) if o else None,
                                     _p(o[1]) if len(o) > 1 else None, _p(y), threads)
        return _from_bits(y)

    def linear_fp16_small_m(self, x, fusion=0, others=(), threads=0):
        """The reference's fp16 small-M microkernel (1..4 tokens, INT4 weights); None where the
        CPU has no AVX512-FP16."""
        xb = _bf16_bits(x)
        m = xb.shape[0]
        n_out = self.n // 2 if fusion == 0x100 else self.n
        y = np.empty((m, n_out), dtype=np.uint16)
        o = [_bf16_bits(t) for t in others]
        rc = lib().woq_oracle_linear_fp16_small_m(self._h, _p(xb), m, fusion, _p(o[0]) if o else None,
                                                  _p(o[1]) if len(o) > 1 else None, _p(y), threads)
        if rc == -2:
            return None
        assert rc == 0, rc
        return _from_bits(y)

    def linear_int8(self, x, fusion=0, others=(), threads=0, want_acc=False):
        xb = _bf16_bits(x)
        m = xb.shape[0]
        n_out = self.n // 2 if fusion == 0x100 else self.n
        y = np.empty((m, n_out), dtype=np.uint16)
        acc = np.empty((m, self.n), dtype=np.int32) if want_acc else None
        o = [_bf16_bits(t) for t in others]
        rc = lib().woq_oracle_linear_int8(self._h, _p(xb), m, fusion, _p(o[0]) if o else None,
                                          _p(o[1]) if len(o) > 1 else None, _p(y), _p(acc), threads)
        assert rc == 0
        return (_from_bits(y), acc) if want_acc else _from_bits(y)


def quant_act_sym(x):
    xb = _bf16_bits(x)
    m, k = xb.shape
    qa = np.empty((m, k), dtype=np.int8)
    sa = np.empty((m,), dtype=np.float32)
    lib().woq_oracle_quant_act_sym(_p(xb), m, k, _p(qa), _p(sa))
    return qa, sa


def max_threads():
    return lib().woq_oracle_max_threads()


def has_fp16_kernel():
    return bool(lib().woq_oracle_has_fp16_kernel())
