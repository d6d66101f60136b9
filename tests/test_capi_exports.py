"""CPU-only: the C-ABI library builds, loads, and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "woq_b200.h")


@pytest.fixture(scope="module")
def built_lib():
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "build_native", os.path.join(ROOT, "intel-extension-for-pytorch_b200", "build_native.py")
    )
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(woq_b200_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("woq_b200_ctx_create", "woq_b200_linear", "woq_b200_ctx_unpack",
                 "woq_b200_dump_dequant", "woq_b200_int8_internals"):
        assert must in syms


def test_library_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/woq_b200.h but not exported"
    lib.woq_b200_version.restype = ctypes.c_int
    assert lib.woq_b200_version() >= 100


def test_python_binding_lists_the_same_symbols(built_lib):
    from ipex_b200 import _capi

    assert sorted(_capi.EXPORTS) == declared_symbols()
    _capi.lib()


def test_bad_arguments_are_rejected_without_a_gpu(built_lib):
    """Argument checks run on the host before any CUDA call."""
    from ipex_b200 import _capi

    L = _capi.lib()
    h = ctypes.c_void_p()
    d = _capi.Desc(n=64, k=64, weight_dtype=_capi.DTYPE_INT4, group_size=0)
    rc = L.woq_b200_ctx_create(ctypes.byref(d), 16, 16, None, None, None, ctypes.byref(h))
    assert rc == 1 and b"group_size" in L.woq_b200_last_error()
    # a valid reference configuration this build lacks: NF4 weights in a GPTQ checkpoint layout
    d = _capi.Desc(n=64, k=64, weight_dtype=_capi.DTYPE_NF4, group_size=64, lowp_mode=_capi.LOWP_BF16,
                   weight_format=_capi.FMT_GPTQ, scale_dtype=_capi.T_F32)
    rc = L.woq_b200_ctx_create(ctypes.byref(d), 16, 16, None, None, None, ctypes.byref(h))
    assert rc == 2
    assert L.woq_b200_ctx_destroy(None) == 1
    assert L.woq_b200_linear(None, None, 1, 64, 0, None, 0, None, 64, None, 0, None) == 1
    fake = (ctypes.c_uint64 * 64)()
    assert L.woq_b200_ctx_destroy(ctypes.cast(fake, ctypes.c_void_p)) == 5


def test_tensor_core_pipeline_shapes_keep_the_ring_rules(built_lib):
    """woq_b200_tc_plan for every token-column count a launch can have: at least four slots in the
    A-group / activation ring (a warpgroup works on every fourth stage), a packed-weight ring whose
    length is a multiple of four (every slot belongs to one warpgroup, which has itself waited for
    the slot's previous use - a parity wait cannot tell one missing completion from three), the A
    groups inside the 512 TMEM columns, the tiles 1024-byte aligned, shared memory within a CTA's
    227 KB."""
    from ipex_b200 import _capi

    for n_tok in range(16, 257, 16):
        p = _capi.tc_plan(n_tok)
        assert p["kbs"] == (3 if n_tok <= 64 else 2 if n_tok <= 128 else 1), (n_tok, p)
        assert p["stages"] >= 4, (n_tok, p)
        assert p["w_ring"] >= 4 and p["w_ring"] % 4 == 0 and p["w_ring"] <= 32, (n_tok, p)
        assert p["a_col0"] >= n_tok and p["a_col0"] % 32 == 0, (n_tok, p)
        assert p["a_col0"] + 32 * p["kbs"] * p["stages"] <= 512, (n_tok, p)
        x_stage = p["kbs"] * n_tok * 128
        w_stage = p["kbs"] * 4096 + (p["kbs"] + 1) * 512
        assert x_stage % 1024 == 0 and w_stage % 16 == 0
        assert p["smem_bytes"] == 1024 + p["stages"] * x_stage + p["w_ring"] * w_stage, (n_tok, p)
        assert p["smem_bytes"] <= 227 * 1024, (n_tok, p)
    assert _capi.tc_plan(256) == {"kbs": 1, "stages": 6, "w_ring": 4, "a_col0": 256, "smem_bytes": 1024 + 6 * 32768 + 4 * 5120}
    assert _capi.tc_plan(128)["stages"] == 4 and _capi.tc_plan(128)["w_ring"] == 8
    L = _capi.lib()
    out = (ctypes.c_int32 * 5)()
    for bad in (0, 8, 24, 272):
        assert L.woq_b200_tc_plan(bad, out) == 1
