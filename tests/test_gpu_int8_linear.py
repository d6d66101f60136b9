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


def make_ctx(capi, layer, flags=0, act_mode=None):
    return capi.WoqContext(torch.from_numpy(layer["qw"]).cuda(), torch.from_numpy(layer["s"]).cuda(),
                           None, None if layer["bias"] is None else torch.from_numpy(layer["bias"]).cuda(),
                           layer["n"], layer["k"], capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                           act_quant_mode=capi.ACT_PER_M_SYM if act_mode is None else act_mode, layout_flags=flags)


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


# The other activation quantisation modes of the reference that share the whole-K accumulators:
# per tensor (0 asymmetric, 4 symmetric) and per token asymmetric (2).  Asymmetric codes are
# unsigned with a zero point, taken out again with the per-row sums of the weight codes.
@pytest.mark.parametrize("act_mode", [0, 2, 4])
@pytest.mark.parametrize("m,n,k", [(1, 96, 256), (8, 640, 1024), (64, 1536, 4096), (300, 640, 1024)])
def test_activation_modes_internals_bit_exact(capi, act_mode, m, n, k):
    layer = make_layer(n, k, seed=5 * n + m + act_mode)
    ctx = make_ctx(capi, layer, act_mode=act_mode)
    x = make_acts(m, k, seed=m + n + act_mode)
    x += 0.37  # a range that is not centred on zero, so the zero points matter
    x = O.rne_bf16(x)
    qa, sa, acc = ctx.int8_internals(bf16_tensor(x, "cuda"))
    zp = ctx.int8_zero_points(m)
    ctx.workspace(m).status()
    qa_ref, sa_ref, zp_ref = O.dynamic_quant(x, act_mode)
    codes = qa.cpu().numpy()
    np.testing.assert_array_equal(codes.view(qa_ref.dtype), qa_ref)
    np.testing.assert_array_equal(sa.cpu().numpy(), sa_ref)
    if zp_ref is None:
        assert not zp.any()
    else:
        np.testing.assert_array_equal(zp.cpu().numpy(), zp_ref)
    np.testing.assert_array_equal(acc.cpu().numpy(), O.int8_accumulators(qa_ref, layer["qw"]))


@pytest.mark.parametrize("act_mode", [0, 2, 4])
@pytest.mark.parametrize("m", [1, 8, 64, 512])
def test_activation_modes_outputs(capi, act_mode, m):
    layer = make_layer(1024, 2048, seed=17 + act_mode, bias=True)
    ctx = make_ctx(capi, layer, act_mode=act_mode)
    x = O.rne_bf16(make_acts(m, 2048, seed=40 + m) + 0.25)
    resid = make_acts(m, 1024, seed=41 + m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_ADD, [bf16_tensor(resid, "cuda")]))
    ctx.workspace(m).status()
    check_tol = O.parity_metrics(y, O.woq_linear_int8(x, layer["qw"], layer["s"], layer["bias"], O.FUSE_ADD, [resid],
                                                      act_mode=act_mode))
    assert check_tol[0] <= O.MAX_ABS_TOL and check_tol[1] <= O.MEAN_REL_TOL, check_tol


def test_asymmetric_gate_up_silu_mul(capi):
    layer = make_layer(1024, 1024, seed=23)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_GATE_UP, act_mode=capi.ACT_PER_M)
    x = O.rne_bf16(make_acts(24, 1024, seed=24) - 0.3)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_SILU_MUL))
    mx, mr = O.parity_metrics(y, O.woq_linear_int8(x, layer["qw"], layer["s"], None, O.FUSE_SILU_MUL,
                                                   act_mode=O.ACT_PER_M))
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


def test_other_int8_recipes_take_their_own_routes(capi):
    """INT8 weights without INT8 compute run on the general kernel, an activation range per K block
    on the K-block INT8 kernel (tests/test_gpu_generic.py, tests/test_gpu_int8_block.py); what no
    kernel takes is refused with a status, never run as something else."""
    layer = make_layer(64, 128, seed=1)
    qw, s = torch.from_numpy(layer["qw"]).cuda(), torch.from_numpy(layer["s"]).cuda()
    assert capi.WoqContext(qw, s, None, None, 64, 128, capi.DTYPE_INT8, -1, capi.LOWP_BF16).route() == capi.ROUTE_GENERAL
    assert capi.WoqContext(qw, s, None, None, 64, 128, capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                           act_quant_mode=7).route() == capi.ROUTE_INT8_BLOCK
    assert capi.WoqContext(qw, s, None, None, 64, 128, capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                           act_quant_mode=6).route() == capi.ROUTE_INT8
    with pytest.raises(capi.WoqError) as e:  # K block of 32: below what the integer kernel takes
        capi.WoqContext(qw[:, :96].contiguous(), s, None, None, 64, 96, capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                        act_quant_mode=7)
    assert e.value.code == 2


# --------------------------------------------------------------------------------------------
# RMSNorm fused with the per-token quantiser; linears on quantised activations


@pytest.mark.parametrize("mode_name", ["PER_M_SYM", "PER_M"])
@pytest.mark.parametrize("m", [1, 7, 300])
def test_rmsnorm_quant_feeds_the_int8_linear(capi, mode_name, m):
    """woq_b200_rmsnorm_quant + woq_b200_linear_prequant against the unfused pair: the
    normalised row is the oracle's rmsnorm (bf16, a last-bit difference allowed where the fp32
    mean differs by summation order), its codes / scales / zero points are bit for bit those of
    the library's own quantiser run on that row, and the linear on the shared codes equals the
    linear that quantises for itself."""
    mode = getattr(capi, "ACT_" + mode_name)
    n, k = 384, 1024
    rng = np.random.default_rng(40 + m)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    qw, s, _ = O.quantize_per_channel(w, O.WOQ_DTYPE_INT8, True)
    ctx = capi.WoqContext(torch.from_numpy(qw).cuda(), torch.from_numpy(s).cuda(), None, None, n, k,
                          capi.DTYPE_INT8, -1, capi.LOWP_INT8, act_quant_mode=mode)
    x = O.rne_bf16((rng.standard_normal((m, k)) * 3.0 + 0.5).astype(np.float32))
    gamma = O.rne_bf16((rng.random(k) + 0.5).astype(np.float32))
    eps = 1e-5
    xg, gg = bf16_tensor(x, "cuda"), bf16_tensor(gamma, "cuda")
    qa, sa, zpa, y = capi.rmsnorm_quant(xg, gg, eps, mode, want_y=True)
    y_ref = O.rmsnorm_bf16(x, gamma, eps)
    y_np = bf16_numpy(y)
    differ = y_np != y_ref
    assert differ.mean() < 2e-3, differ.mean()
    np.testing.assert_allclose(y_np, y_ref, rtol=2.0 ** -7, atol=0)
    # the library's own quantiser on the same normalised rows
    qa2, sa2, _ = ctx.int8_internals(y)
    assert torch.equal(qa, qa2) and torch.equal(sa, sa2)
    if mode == capi.ACT_PER_M:
        assert torch.equal(zpa, ctx.int8_zero_points(m))
    else:
        assert zpa is None
    # the linear on the shared codes equals the linear that quantises for itself
    want = ctx.linear(y)
    got = ctx.linear_prequant(qa, sa, zpa)
    assert torch.equal(got, want)
    resid = bf16_tensor(rng.standard_normal((m, n)).astype(np.float32), "cuda")
    assert torch.equal(ctx.linear_prequant(qa, sa, zpa, capi.FUSE_ADD, [resid]), ctx.linear(y, capi.FUSE_ADD, [resid]))
    # and the whole thing against the oracle
    ref = O.woq_linear_int8(y_np, qw, s, None, act_mode=mode)
    mx, mr = O.parity_metrics(bf16_numpy(got), ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


def test_rmsnorm_quant_rejects_what_it_cannot_do(capi):
    x = torch.zeros((2, 64), dtype=torch.bfloat16, device="cuda")
    g = torch.ones((64,), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.WoqError, match="per token"):
        capi.rmsnorm_quant(x, g, 1e-5, capi.ACT_PER_TENSOR_SYM)
    with pytest.raises(capi.WoqError, match="multiple of 16"):
        capi.rmsnorm_quant(x[:, :40].contiguous(), g[:40].contiguous(), 1e-5, capi.ACT_PER_M_SYM)
    # a context that quantises per K block cannot take per-token codes
    w = (np.random.default_rng(0).standard_normal((64, 128)) * 0.02).astype(np.float32)
    qw, s, _ = O.quantize_per_channel(w, O.WOQ_DTYPE_INT8, True)
    blk = capi.WoqContext(torch.from_numpy(qw).cuda(), torch.from_numpy(s).cuda(), None, None, 64, 128,
                          capi.DTYPE_INT8, -1, capi.LOWP_INT8, act_quant_mode=capi.ACT_PER_M_K_BLOCK_SYM)
    qa = torch.zeros((2, 128), dtype=torch.int8, device="cuda")
    sa = torch.ones((2,), dtype=torch.float32, device="cuda")
    with pytest.raises(capi.WoqError, match="tcgen05 INT8 route"):
        blk.linear_prequant(qa, sa)
