"""GPU parity of the INT4 WOQ linear (lowp BF16) against the CPU oracle, through the C ABI.

Bars: repack round trip and dequantised weights bit-exact; bf16 outputs within
max-abs <= 1e-2 * ||y_ref||_inf and mean relative error <= 2e-3.
"""
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


def make_ctx(capi, layer, flags=0, hint=0):
    qw, s, z, b = to_device_layer(layer, "cuda")
    return capi.WoqContext(qw, s, z, b, layer["n"], layer["k"], capi.DTYPE_INT4, layer["g"],
                           capi.LOWP_BF16, layout_flags=flags, kernel_hint=hint)


def oracle_y(layer, x, fusion=O.FUSE_NONE, others=()):
    return O.woq_linear_bf16(x, layer["qw"], layer["s16"], layer["z"], layer["bias"],
                             O.WOQ_DTYPE_INT4, layer["g"], fusion, others)


def assert_parity(y, y_ref):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL, f"max-abs/inf-norm {mx:.3e}"
    assert mr <= O.MEAN_REL_TOL, f"mean rel {mr:.3e}"


@pytest.mark.parametrize("n,k,g", [(64, 64, 64), (100, 256, 128), (500, 512, 128), (4096, 4096, 128),
                                   (192, 1024, -1), (128, 1024, 256), (64, 2048, 1024)])
def test_repack_round_trip_bit_exact(capi, n, k, g):
    layer = make_int4_layer(n, k, g, seed=n + k)
    ctx = make_ctx(capi, layer)
    back = ctx.unpack().cpu().numpy()
    np.testing.assert_array_equal(back, layer["qw"])


@pytest.mark.parametrize("n,k,g,sym", [(100, 256, 128, False), (512, 1024, 64, False),
                                       (4096, 4096, 128, False), (256, 512, -1, False),
                                       (128, 512, 128, True)])
def test_dequantised_weights_bit_exact(capi, n, k, g, sym):
    layer = make_int4_layer(n, k, g, seed=7 * n + k, sym=sym)
    ctx = make_ctx(capi, layer)
    w = bf16_numpy(ctx.dump_dequant())
    w_ref = O.dequantize_weight(layer["qw"], layer["s16"], layer["z"], O.WOQ_DTYPE_INT4, k, g)
    np.testing.assert_array_equal(w.view(np.uint32), w_ref.view(np.uint32))


@pytest.mark.parametrize("m", [1, 3, 8, 16])
@pytest.mark.parametrize("n,k,g,std", [(256, 512, 128, 0.02), (192, 1024, 64, 0.02), (128, 768, -1, 0.02),
                                       (256, 512, 128, 3.0), (128, 512, 256, 1e-3)])
def test_decode_kernels_use_the_exact_dequantised_weights(capi, m, n, k, g, std):
    """A one-hot activation row picks out one column of the dequantised weight, so the decode
    kernels' own dequantisers (every nibble position, both small and large scales) must
    reproduce bf16((q - zp) * bf16(scale)) bit for bit."""
    layer = make_int4_layer(n, k, g, seed=n + k + m, std=std)
    ctx = make_ctx(capi, layer)
    w_ref = O.dequantize_weight(layer["qw"], layer["s16"], layer["z"], O.WOQ_DTYPE_INT4, k, g)
    rng = np.random.default_rng(m)
    for start in range(0, 64, m):
        cols = [(start + i) * (k // 64) % k + (start + i) % 64 for i in range(m)]
        cols = [c % k for c in cols]
        x = np.zeros((m, k), np.float32)
        x[np.arange(m), cols] = 1.0
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
        np.testing.assert_array_equal(y.view(np.uint32), w_ref[:, cols].T.copy().view(np.uint32))
    ctx.workspace(m).status()


@pytest.mark.parametrize("m", [1, 4, 32, 256])
def test_config1_single_linear(capi, m):
    """N = K = 4096, INT4 asymmetric, group 128, no bias, M in {1, 4, 32, 256}."""
    layer = make_int4_layer(4096, 4096, 128, seed=1000)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, 4096, seed=1000 + m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    assert_parity(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 13, 16, 17, 40])
@pytest.mark.parametrize("n,k,g", [(64, 64, 64), (200, 320, 64), (768, 1536, 128), (96, 3584, 128),
                                   (1280, 1024, -1), (320, 2048, 512)])
def test_shapes_and_ragged_m(capi, m, n, k, g):
    layer = make_int4_layer(n, k, g, seed=n * 3 + k + m, bias=(n % 128 != 0))
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    assert_parity(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [1, 8, 16])
def test_scale_after_sum_variant_within_tolerance(capi, m):
    """HINT_STREAM_FAST skips the per-weight bf16 rounding; it must still meet the output bar."""
    layer = make_int4_layer(4096, 4096, 128, seed=1000)
    ctx = make_ctx(capi, layer, hint=capi.HINT_STREAM_FAST)
    x = make_acts(m, 4096, seed=1000 + m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    assert_parity(y, oracle_y(layer, x))


def test_m_zero_returns_empty(capi):
    layer = make_int4_layer(64, 64, 64, seed=3)
    ctx = make_ctx(capi, layer)
    y = ctx.linear(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"))
    assert tuple(y.shape) == (0, 64)


FUSIONS = [
    (O.FUSE_GELU_ERF, 0), (O.FUSE_GELU_TANH, 0), (O.FUSE_RELU, 0), (O.FUSE_SILU, 0),
    (O.FUSE_ADD, 1), (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1),
]


@pytest.mark.parametrize("fusion,n_others", FUSIONS)
@pytest.mark.parametrize("m", [4, 16])
def test_fused_post_ops(capi, fusion, n_others, m):
    layer = make_int4_layer(640, 1024, 128, seed=fusion + 11, std=0.05, bias=True)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, 1024, seed=fusion)
    others = [make_acts(m, 640, seed=50 + i) for i in range(n_others)]
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), fusion, [bf16_tensor(o, "cuda") for o in others]))
    assert_parity(y, oracle_y(layer, x, fusion, others))


@pytest.mark.parametrize("m", [1, 7, 16])
def test_gate_up_silu_mul(capi, m):
    """Fused gate/up: equals woq_linear_silu then woq_linear_mul of the reference."""
    inter, k = 1792, 1024
    layer = make_int4_layer(2 * inter, k, 128, seed=77, std=0.05)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_GATE_UP)
    # the interleaved layout still unpacks / dequantises to the caller's row order
    np.testing.assert_array_equal(ctx.unpack().cpu().numpy(), layer["qw"])
    x = make_acts(m, k, seed=m + 5)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_SILU_MUL))
    assert y.shape == (m, inter)
    assert_parity(y, oracle_y(layer, x, O.FUSE_SILU_MUL))
    # two-op composition through separate contexts gives the same numbers
    half = {**layer, "qw": layer["qw"][:inter], "s16": layer["s16"][:inter], "z": layer["z"][:inter], "n": inter}
    up = {**layer, "qw": layer["qw"][inter:], "s16": layer["s16"][inter:], "z": layer["z"][inter:], "n": inter}
    cg, cu = make_ctx(capi, half), make_ctx(capi, up)
    xg = bf16_tensor(x, "cuda")
    t = cg.linear(xg, capi.FUSE_SILU)
    y2 = bf16_numpy(cu.linear(xg, capi.FUSE_MUL, [t]))
    assert_parity(y2, oracle_y(layer, x, O.FUSE_SILU_MUL))
    assert (y == y2).mean() > 0.95  # same weights, different split of K: a few last-bit flips


def test_results_do_not_depend_on_timing(capi):
    """Split-K partials are reduced in a fixed order: repeated calls are bit-identical."""
    layer = make_int4_layer(4096, 4096, 128, seed=5)
    ctx = make_ctx(capi, layer)
    x = bf16_tensor(make_acts(8, 4096, seed=9), "cuda")
    y0 = ctx.linear(x).clone()
    for _ in range(5):
        assert torch.equal(ctx.linear(x), y0)


def test_linearity_at_full_size(capi):
    """Llama-3-70B gate_up shard shape; size-independent property: y(2x) == 2*y(x) exactly
    (scaling by two is exact in every format on the path)."""
    n, k = 7168, 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    qw = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda", generator=g)
    s = (torch.rand((n, k // 128), device="cuda", generator=g) * 0.01 + 0.001).half()
    z = torch.randint(0, 16, (n, k // 128), device="cuda", generator=g).float()
    ctx = capi.WoqContext(qw, s, z, None, n, k, capi.DTYPE_INT4, 128, capi.LOWP_BF16)
    assert torch.equal(ctx.unpack(), qw)
    x = torch.randn((4, k), device="cuda", generator=g).bfloat16()
    y1 = ctx.linear(x).float()
    y2 = ctx.linear(x * 2).float()
    assert torch.equal(y2, 2 * y1)
    # against a plain torch fp32 matmul on the dumped weights
    w = ctx.dump_dequant().float()
    y_ref = (x.float() @ w.T).bfloat16().float()
    mx, mr = O.parity_metrics(y1.cpu().numpy(), y_ref.cpu().numpy())
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL


def test_awq_checkpoint_fixture(capi, golden_dir):
    """AWQ int32 checkpoint tensors of the reference's test data, ingested on the device."""
    import os

    f = np.load(os.path.join(golden_dir, "awq_fixture.npz"))
    k, n = f["qweight"].shape[0], f["qweight"].shape[1] * 8
    qweight = torch.from_numpy(f["qweight"]).cuda()
    qzeros = torch.from_numpy(f["qzeros"]).cuda()
    scales = bf16_tensor(O.from_bf16_bits(f["scales_bf16"]), "cuda")
    bias = bf16_tensor(O.from_bf16_bits(f["bias_bf16"]), "cuda")
    ctx = capi.WoqContext(qweight, scales, qzeros, bias, n, k, capi.DTYPE_INT4, 128, capi.LOWP_BF16,
                          weight_format=capi.FMT_AWQ)
    qw_ref, s_ref, z_ref = O.awq_to_plain(f["qweight"], f["qzeros"], O.from_bf16_bits(f["scales_bf16"]))
    np.testing.assert_array_equal(ctx.unpack().cpu().numpy(), qw_ref)
    w = bf16_numpy(ctx.dump_dequant())
    w_ref = O.dequantize_weight(qw_ref, s_ref, z_ref, O.WOQ_DTYPE_INT4, k, 128)
    np.testing.assert_array_equal(w.view(np.uint32), w_ref.view(np.uint32))
    x = O.from_bf16_bits(f["act_bf16"])
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    y_gold = O.from_bf16_bits(f["y_ref_bf16"])
    assert np.abs(y - y_gold).max() <= 0.1  # the reference test's own tolerance


def test_errors_are_reported_not_thrown_from_kernels(capi):
    layer = make_int4_layer(64, 128, 64, seed=1)
    ctx = make_ctx(capi, layer)
    x = torch.zeros((2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.WoqError) as e:
        ctx.linear(x, capi.FUSE_ADD, [])
    assert e.value.code == 1
    with pytest.raises(capi.WoqError) as e:
        ctx.linear(x, capi.FUSE_SILU_MUL)
    assert e.value.code == 1
    small = capi.Workspace(16, "cuda")
    with pytest.raises(capi.WoqError) as e:
        ctx.linear(x, workspace=small)
    assert e.value.code == 4
    zbad = torch.full((64, 2), 3.5, device="cuda")
    qw, s, _, _ = to_device_layer(layer, "cuda")
    with pytest.raises(capi.WoqError):
        capi.WoqContext(qw, s, zbad, None, 64, 128, capi.DTYPE_INT4, 64, capi.LOWP_BF16)


def test_strided_output_takes_operands_with_the_same_row_stride(capi):
    """y rows and the rows of the fused operands share one stride (ldy).  A column slice of a
    wider buffer as output works with a residual sliced the same way; a dense residual beside a
    strided output is refused by the ctypes layer instead of being read with the wrong stride."""
    n, k, m = 320, 512, 6
    layer = make_int4_layer(n, k, 128, seed=91, std=0.05)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=92)
    r = make_acts(m, n, seed=93)
    wide_out = torch.zeros((m, 2 * n), dtype=torch.bfloat16, device="cuda")
    wide_res = torch.zeros((m, 2 * n), dtype=torch.bfloat16, device="cuda")
    wide_res[:, n:] = bf16_tensor(r, "cuda")
    ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_ADD, [wide_res[:, n:]], out=wide_out[:, n:])
    assert_parity(bf16_numpy(wide_out[:, n:]), oracle_y(layer, x, O.FUSE_ADD, [r]))
    assert not wide_out[:, :n].any()
    with pytest.raises(ValueError, match="row stride"):
        ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_ADD, [bf16_tensor(r, "cuda")], out=wide_out[:, n:])


def test_deferred_zero_point_check_reports_at_first_use(capi):
    layer = make_int4_layer(64, 128, 64, seed=1)
    qw, s, _, _ = to_device_layer(layer, "cuda")
    zbad = torch.full((64, 2), 3.5, device="cuda")
    ctx = capi.WoqContext(qw, s, zbad, None, 64, 128, capi.DTYPE_INT4, 64, capi.LOWP_BF16,
                          layout_flags=capi.LAYOUT_DEFER_CHECK)
    x = torch.zeros((2, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.WoqError) as e:
        ctx.linear(x)
    assert e.value.code == 1 and "zero points" in str(e.value)
    good = capi.WoqContext(*to_device_layer(layer, "cuda")[:3], None, 64, 128, capi.DTYPE_INT4, 64,
                           capi.LOWP_BF16, layout_flags=capi.LAYOUT_DEFER_CHECK)
    y = bf16_numpy(good.linear(bf16_tensor(make_acts(2, 128, seed=3), "cuda")))
    assert_parity(y, oracle_y(layer, make_acts(2, 128, seed=3)))
