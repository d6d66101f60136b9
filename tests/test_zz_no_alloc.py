"""The allocation-free entry point, checked against the regular one.

woq_b200_linear_static_scratch exists for hosts that cannot allocate device memory when they run
a linear (a memory planner owns every byte, a server forbids allocation after start-up, a
sandboxed allocator is not re-entrant): it uses a scratch array built into the library instead of
a caller-provided workspace.  It must give the same numbers as woq_b200_linear, also on a second
call that finds the previous call's leftovers in the array.  This file sorts last on purpose, so a
run that stops at the first failure has already been through every other test."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, make_acts, make_int4_layer, to_device_layer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ipex_b200 import _capi

    _capi.lib()
    return _capi


@pytest.mark.parametrize("split", ["stream_k", "auto"])
def test_two_calls_in_a_row_match_the_regular_entry_point(capi, split):
    """With the stream-K split forced, K is shared between thread blocks through the scratch
    (partial tiles and arrival counters live in the built-in array); with the library's own
    choice this layer reduces inside thread-block clusters and only the status word is used."""
    n, k, g = 1536, 4096, 128
    layer = make_int4_layer(n, k, g, seed=4242, bias=True)
    qw, s, z, b = to_device_layer(layer, "cuda")
    ctx = capi.WoqContext(qw, s, z, b, n, k, capi.DTYPE_INT4, g, capi.LOWP_BF16)
    capi.set_option(capi.OPT_DECODE_SPLIT, capi.SPLIT_STREAM_K if split == "stream_k" else capi.SPLIT_AUTO)
    try:
        _two_calls(capi, ctx, layer, n, k, g)
    finally:
        capi.set_option(capi.OPT_DECODE_SPLIT, capi.SPLIT_AUTO)


def _two_calls(capi, ctx, layer, n, k, g):

    # call 1: plain linear, 3 tokens
    x1 = make_acts(3, k, seed=1)
    y_regular = ctx.linear(bf16_tensor(x1, "cuda"))
    y_static = ctx.linear_static_scratch(bf16_tensor(x1, "cuda"))
    torch.cuda.synchronize()
    assert torch.equal(y_static, y_regular)            # same kernel, same split: bit-identical
    y_ref = O.woq_linear_bf16(x1, layer["qw"], layer["s16"], layer["z"], layer["bias"],
                              O.WOQ_DTYPE_INT4, g)
    mx, mr = O.parity_metrics(bf16_numpy(y_static), y_ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)

    # call 2, straight after: other inputs, 16 tokens, a fused residual add
    x2 = make_acts(16, k, seed=2)
    r2 = make_acts(16, n, seed=3)
    y_regular2 = ctx.linear(bf16_tensor(x2, "cuda"), capi.FUSE_ADD, [bf16_tensor(r2, "cuda")])
    y_static2 = ctx.linear_static_scratch(bf16_tensor(x2, "cuda"), capi.FUSE_ADD, [bf16_tensor(r2, "cuda")])
    torch.cuda.synchronize()
    assert torch.equal(y_static2, y_regular2)
    y_ref2 = O.woq_linear_bf16(x2, layer["qw"], layer["s16"], layer["z"], layer["bias"],
                               O.WOQ_DTYPE_INT4, g, O.FUSE_ADD, [r2])
    mx, mr = O.parity_metrics(bf16_numpy(y_static2), y_ref2)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)
    capi.static_scratch_status()       # no kernel gave up a wait

    # call 3: everything pre-allocated by the caller -> the library allocates nothing
    xg, rg = bf16_tensor(x2, "cuda"), bf16_tensor(r2, "cuda")
    out = torch.empty((16, n), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    ctx.linear_static_scratch(xg, capi.FUSE_ADD, [rg], out=out)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == allocated_before
    assert torch.equal(out, y_regular2)


def test_sizes_beyond_the_built_in_scratch_are_refused(capi):
    layer = make_int4_layer(64, 128, 64, seed=1)
    qw, s, z, b = to_device_layer(layer, "cuda")
    ctx = capi.WoqContext(qw, s, z, b, 64, 128, capi.DTYPE_INT4, 64, capi.LOWP_BF16)
    x = torch.zeros((17, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.WoqError) as e:
        ctx.linear_static_scratch(x)
    assert e.value.code == 1 and "at most 16 tokens" in str(e.value)
    L = capi.lib()
    assert L.woq_b200_linear_static_scratch(None, None, 1, 128, 0, None, 0, None, 64, None) == 5
