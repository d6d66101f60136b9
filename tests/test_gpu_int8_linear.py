"""GPU parity of the INT8-compute path (INT8 symmetric per-channel weights, per-token symmetric
int8 activations, int32 accumulation) against the CPU oracle, through the C ABI.

Bars: repack round trip, activation codes / scales and int32 accumulators bit-exact; bf16
outputs within max-abs <= 1e-2 * ||y_ref||_inf and mean relative error <= 2e-3."""
import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, make_acts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ipex_b200 import _capi

    _capi.lib()
    return _capi


def make_layer(n, k, seed, bias=False):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    qw, s, _ = O.quantize_per_channel(w, O.WOQ_DTYPE_INT8, sym=True)
    b = (rng.standard_normal(n) * 0.1).astype(np.float32) if bias else None
    return dict(qw=qw, s=s, bias=b, n=n, k=k)


def make_ctx(capi, layer, flags=0):
    return capi.WoqContext(torch.from_numpy(layer["qw"]).cuda(), torch.from_numpy(layer["s"]).cuda(),
                           None, None if layer["bias"] is None else torch.from_numpy(layer["bias"]).cuda(),
                           layer["n"], layer["k"], capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                           act_quant_mode=capi.ACT_PER_M_SYM, layout_flags=flags)


def check(y, y_ref):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)
    assert (y == y_ref).mean() > 0.99  # exact integer sums; only the last fp32 steps may differ


@pytest.mark.parametrize("n,k", [(64, 128), (100, 256), (500, 1024), (4096, 4096)])
def test_repack_round_trip_bit_exact(capi, n, k):
    layer = make_layer(n, k, seed=n + k)
    ctx = make_ctx(capi, layer)
    np.testing.assert_array_equal(ctx.unpack().cpu().numpy(), layer["qw"])


@pytest.mark.parametrize("m", [1, 8, 64, 300])
@pytest.mark.parametrize("n,k", [(96, 256), (640, 1024), (1536, 4096)])
def test_internals_bit_exact(capi, m, n, k):
    layer = make_layer(n, k, seed=3 * n + m)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=m + n)
    if m > 2:
        x[1] = 0.0  # a row of zeros: scale 0, codes 0
    qa, sa, acc = ctx.int8_internals(bf16_tensor(x, "cuda"))
    ctx.workspace(m).status()
    qa_ref, sa_ref, _ = O.dynamic_quant_per_token(x, sym=True)
    np.testing.assert_array_equal(qa.cpu().numpy(), qa_ref)
    np.testing.assert_array_equal(sa.cpu().numpy(), sa_ref)
    np.testing.assert_array_equal(acc.cpu().numpy(), O.int8_accumulators(qa_ref, layer["qw"]))


@pytest.mark.parametrize("m", [1, 8, 64, 512])
def test_config2_qkv_and_o_proj(capi, m):
    for n, k, seed in ((6144, 4096, 2000), (4096, 4096, 2001)):
        layer = make_layer(n, k, seed=seed)
        ctx = make_ctx(capi, layer)
        x = make_acts(m, k, seed=seed + m)
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
        ctx.workspace(m).status()
        check(y, O.woq_linear_int8(x, layer["qw"], layer["s"], None))


@pytest.mark.parametrize("m", [1, 8, 64])
def test_config2_gate_up_silu_mul(capi, m):
    n, k = 28672, 4096
    layer = make_layer(n, k, seed=2002)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_GATE_UP)
    x = make_acts(m, k, seed=2002 + m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_SILU_MUL))
    assert y.shape == (m, n // 2)
    mx, mr = O.parity_metrics(y, O.woq_linear_int8(x, layer["qw"], layer["s"], None, O.FUSE_SILU_MUL))
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


@pytest.mark.parametrize("m", [1, 8, 64, 512])
def test_config2_down_proj_add(capi, m):
    n, k = 4096, 14336
    layer = make_layer(n, k, seed=2003, bias=True)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=2003 + m)
    r = make_acts(m, n, seed=7)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_ADD, [bf16_tensor(r, "cuda")]))
    check(y, O.woq_linear_int8(x, layer["qw"], layer["s"], layer["bias"], O.FUSE_ADD, [r]))


@pytest.mark.parametrize("fusion,n_others", [(O.FUSE_GELU_ERF, 0), (O.FUSE_RELU, 0), (O.FUSE_SILU, 0),
                                             (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1)])
def test_fused_post_ops(capi, fusion, n_others):
    n, k, m = 640, 1024, 20
    layer = make_layer(n, k, seed=fusion, bias=True)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=fusion + 1)
    others = [make_acts(m, n, seed=30 + i) for i in range(n_others)]
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), fusion, [bf16_tensor(o, "cuda") for o in others]))
    mx, mr = O.parity_metrics(y, O.woq_linear_int8(x, layer["qw"], layer["s"], layer["bias"], fusion, others))
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


def test_unsupported_modes_are_reported(capi):
    layer = make_layer(64, 128, seed=1)
    qw, s = torch.from_numpy(layer["qw"]).cuda(), torch.from_numpy(layer["s"]).cuda()
    with pytest.raises(capi.WoqError) as e:
        capi.WoqContext(qw, s, None, None, 64, 128, capi.DTYPE_INT8, -1, capi.LOWP_BF16)
    assert e.value.code == 2
    with pytest.raises(capi.WoqError) as e:
        capi.WoqContext(qw, s, None, None, 64, 128, capi.DTYPE_INT8, -1, capi.LOWP_INT8, act_quant_mode=2)
    assert e.value.code == 2
