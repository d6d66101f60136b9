"""The general route (woq_b200_linear_any): every weight dtype and every floating compute dtype
the reference routes (csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:75-165), shapes off the 64-element
grid, against the CPU oracle.

Bars: the values the kernel multiplies by (woq_b200_dump_dequant_f32) bit-exact; outputs within
max-abs <= 1e-2 * ||y_ref||_inf and mean relative error <= 2e-3 for bf16 / fp16 compute, and
within 2e-5 / 2e-5 for fp32 compute (summation order only)."""
import copy

import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import make_acts

pytestmark = pytest.mark.gpu
TORCH = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


@pytest.fixture(scope="module")
def ipex():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ipex_b200

    ipex_b200.load_ops()
    return ipex_b200


def make_layer(kind, n, k, g, seed):
    """(codes, scales, zps, weight dtype code) as the reference's quantiser / a checkpoint gives them."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if kind == "fp8":
        codes = rng.integers(0, 256, (n, k), dtype=np.uint8)
        codes[(codes & 0x7F) == 0x7F] = 0x3A  # keep clear of the NaN patterns of e4m3
        codes[(codes & 0x78) == 0x78] &= 0xBF  # and of the largest magnitudes
        s = (rng.random((n, 1 if g <= 0 else -(-k // g)), dtype=np.float32) * 0.01 + 0.001).astype(np.float32)
        return codes, s, None, O.WOQ_DTYPE_FP8
    dt = {"int4": O.WOQ_DTYPE_INT4, "int4_sym": O.WOQ_DTYPE_INT4, "nf4": O.WOQ_DTYPE_NF4,
          "int8": O.WOQ_DTYPE_INT8, "int8_sym": O.WOQ_DTYPE_INT8}[kind]
    sym = kind in ("int4_sym", "nf4", "int8_sym")
    if g > 0:
        qw, s, z = O.quantize_per_block(w, dt, g, sym)
    else:
        qw, s, z = O.quantize_per_channel(w, dt, sym)
        s = s[:, None]
        z = None if z is None else z[:, None]
    return qw, s, z, dt


def make_ctx(capi, qw, s, z, dt, n, k, g, lowp, bias=None):
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    return capi.WoqContext(t(qw.view(np.uint8) if dt == O.WOQ_DTYPE_FP8 else qw), t(s), t(z), t(bias), n, k, dt, g,
                           lowp, layout_flags=capi.LAYOUT_GENERIC)


def to_io(a, io):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(TORCH[io]).cuda()


def round_io(a, io):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(TORCH[io]).float().numpy()


def check(y, ref, compute):
    mx, mr = O.parity_metrics(y, ref)
    if compute == "fp32":
        assert mx <= 2e-5 and mr <= 2e-5, (mx, mr)
    else:
        assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


CASES = [
    # kind, n, k, group
    ("int4", 96, 512, 128), ("int4", 100, 200, -1), ("int4", 72, 256, 32), ("int4_sym", 64, 320, 64),
    ("int4", 130, 1000, 128), ("nf4", 96, 256, 64), ("nf4", 40, 200, -1),
    ("int8", 80, 384, -1), ("int8_sym", 64, 512, 128), ("fp8", 64, 256, -1), ("fp8", 48, 512, 128),
]


@pytest.mark.parametrize("compute", ["bf16", "fp16", "fp32"])
@pytest.mark.parametrize("kind,n,k,g", CASES)
def test_weights_and_outputs(ipex, kind, n, k, g, compute):
    capi = ipex._capi
    qw, s, z, dt = make_layer(kind, n, k, g, seed=n + k)
    lowp = {"bf16": capi.LOWP_BF16, "fp16": capi.LOWP_FP16, "fp32": capi.LOWP_NONE}[compute]
    rng = np.random.default_rng(k)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32) if n % 3 == 0 else None
    ctx = make_ctx(capi, qw, s, z, dt, n, k, g, lowp, bias)
    assert ctx.route() == capi.ROUTE_GENERAL
    np.testing.assert_array_equal(ctx.unpack().cpu().numpy().view(np.uint8), np.ascontiguousarray(qw).view(np.uint8))
    # the weights the kernel multiplies by
    w = ctx.dump_dequant_f32(TORCH[compute]).cpu().numpy()
    G = k if g <= 0 else g
    q = O.weight_integers(qw, dt, k)
    zz = (8.0 if dt == O.WOQ_DTYPE_INT4 else 0.0) if z is None else O._expand_groups(z, k, G)
    w_ref = O._round_to(((q - zz) * O._expand_groups(O._round_to(s, compute), k, G)).astype(np.float32), compute)
    np.testing.assert_array_equal(w.view(np.uint32), w_ref.view(np.uint32))
    # lowp NONE: the activation's dtype is the compute dtype; otherwise try an io dtype that differs too
    for io in ([compute] if compute == "fp32" else [compute, "fp32"]):
        for m in (1, 9, 21):
            x = round_io(make_acts(m, k, seed=m), io)
            y = ctx.linear_any(to_io(x, io)).float().cpu().numpy()
            check(y, O.woq_linear_any(x, qw, s, z, bias, dt, g, compute, io), compute)


@pytest.mark.parametrize("fusion,n_others", [(O.FUSE_GELU_ERF, 0), (O.FUSE_GELU_TANH, 0), (O.FUSE_RELU, 0),
                                             (O.FUSE_SILU, 0), (O.FUSE_ADD, 1), (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1)])
@pytest.mark.parametrize("io", ["bf16", "fp16", "fp32"])
def test_post_ops(ipex, fusion, n_others, io):
    capi = ipex._capi
    n, k, g, m = 96, 384, 128, 7
    qw, s, z, dt = make_layer("int8", n, k, g, seed=fusion)
    bias = np.linspace(-1, 1, n).astype(np.float32)
    lowp = {"bf16": capi.LOWP_BF16, "fp16": capi.LOWP_FP16, "fp32": capi.LOWP_NONE}[io]
    ctx = make_ctx(capi, qw, s, z, dt, n, k, g, lowp, bias)
    x = round_io(make_acts(m, k, seed=fusion + 1), io)
    others = [round_io(make_acts(m, n, seed=40 + i), io) for i in range(n_others)]
    y = ctx.linear_any(to_io(x, io), fusion, [to_io(o, io) for o in others]).float().cpu().numpy()
    check(y, O.woq_linear_any(x, qw, s, z, bias, dt, g, io, io, fusion, others), io)


def test_reference_edge_shape_9_4095_4095(ipex):
    """The reference's own odd shape (tests/cpu/test_quantization_default_recipe.py:262-316)."""
    capi = ipex._capi
    n = k = 4095
    m = 9
    qw, s, z, dt = make_layer("int4", n, k, 128, seed=9)
    ctx = make_ctx(capi, qw, s, z, dt, n, k, 128, capi.LOWP_BF16)
    x = make_acts(m, k, seed=3)
    y = ctx.linear_any(to_io(x, "bf16")).float().cpu().numpy()
    rows = np.arange(0, n, 7)
    check(y[:, rows], O.woq_linear_any(x, qw[rows], s[rows], z[rows], None, dt, 128, "bf16", "bf16"), "bf16")
    # woq_b200_linear reaches the same route for a context the tuned kernels do not take
    auto = capi.WoqContext(torch.from_numpy(qw).cuda(), torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(), None,
                           n, k, dt, 128, capi.LOWP_BF16)
    assert auto.route() == capi.ROUTE_GENERAL
    assert torch.equal(auto.linear(to_io(x, "bf16")), ctx.linear_any(to_io(x, "bf16")))


def make_linear(n, k, bias, seed):
    torch.manual_seed(seed)
    lin = torch.nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    return lin


def test_default_qconfig_runs(ipex):
    """get_weight_only_quant_qconfig_mapping() with its defaults is INT8 weights (asymmetric, per
    channel) and lowp NONE (intel_extension_for_pytorch/quantization/_qconfig.py:189-307)."""
    q = ipex.quantization
    lin = make_linear(192, 320, True, seed=5)
    w = lin.weight.detach().float().numpy().copy()
    b = lin.bias.detach().float().numpy().copy()
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping().global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    qw, s, z = O.quantize_per_channel(w, O.WOQ_DTYPE_INT8, False)
    for io in ("bf16", "fp16", "fp32"):
        x = round_io(make_acts(6, 320, seed=8), io)
        y = mod(to_io(x, io))
        assert y.dtype == TORCH[io]
        ref = O.woq_linear_any(x, qw, s[:, None], z[:, None], b, O.WOQ_DTYPE_INT8, -1, io, io)
        check(y.float().cpu().numpy(), ref, io)


def test_lowp_none_and_fp16_on_an_int4_layer(ipex):
    """lowp NONE computes in the activation's dtype: bf16 activations take the tuned kernels, fp32
    and fp16 ones the general kernel on a second packing of the layer; lowp FP16 computes in fp16."""
    q = ipex.quantization
    lin = make_linear(256, 512, False, seed=6)
    w = lin.weight.detach().float().numpy().copy()
    qw, s, z = O.quantize_per_block(w, O.WOQ_DTYPE_INT4, 128)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.NONE, group_size=128).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(copy.deepcopy(lin))
    for io in ("bf16", "fp32", "fp16"):
        x = round_io(make_acts(5, 512, seed=2), io)
        y = mod(to_io(x, io))
        assert y.dtype == TORCH[io]
        check(y.float().cpu().numpy(), O.woq_linear_any(x, qw, s, z, None, O.WOQ_DTYPE_INT4, 128, io, io), io)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.FP16, group_size=128).global_qconfig
    mod16 = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(copy.deepcopy(lin))
    x = make_acts(5, 512, seed=2)
    y = mod16(to_io(x, "bf16"))
    check(y.float().cpu().numpy(), O.woq_linear_any(x, qw, s, z, None, O.WOQ_DTYPE_INT4, 128, "fp16", "bf16"), "fp16")


def test_nf4_module(ipex):
    q = ipex.quantization
    lin = make_linear(128, 256, True, seed=7)
    w = lin.weight.detach().float().numpy().copy()
    b = lin.bias.detach().float().numpy().copy()
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.NF4, lowp_mode=q.WoqLowpMode.BF16, group_size=64).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    qw, s, _ = O.quantize_per_block(w, O.WOQ_DTYPE_NF4, 64, True)
    np.testing.assert_array_equal(mod._op_context.get_weight().cpu().numpy(), qw)
    x = make_acts(4, 256, seed=1)
    y = mod(to_io(x, "bf16"))
    check(y.float().cpu().numpy(), O.woq_linear_any(x, qw, s, None, b, O.WOQ_DTYPE_NF4, 64, "bf16", "bf16"), "bf16")


@pytest.mark.parametrize("act_dtype", ["fp32", "bf16"])
def test_default_recipe_runs_end_to_end(ipex, act_dtype):
    """get_weight_only_quant_qconfig_mapping() with no arguments - INT8 weights per channel, lowp
    NONE (compute in the activation's dtype) - and the default INT8-compute recipe (INT8 weights,
    activation mode PER_BATCH_IC_BLOCK_SYM) both build and run through from_float
    (reference: tests/cpu/test_quantization_default_recipe.py:318-419)."""
    q = ipex.quantization
    torch.manual_seed(3)
    lin = torch.nn.Linear(384, 192, bias=True)
    x = torch.randn(5, 384)
    y_fp = lin(x)
    for qmap in (q.get_weight_only_quant_qconfig_mapping(),
                 q.get_weight_only_quant_qconfig_mapping(lowp_mode=q.WoqLowpMode.INT8)):
        mod = copy.deepcopy(lin)
        mod.qconfig = qmap.global_qconfig
        w = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(mod)
        xin = x.to(TORCH[act_dtype]).cuda()
        y = w(xin)
        assert y.dtype == TORCH[act_dtype] and y.shape == (5, 192)
        # 8-bit weights (and 8-bit activations in the second recipe): close to the float layer
        assert torch.nn.functional.cosine_similarity(y.float().cpu().flatten(), y_fp.flatten(), dim=0) > 0.999
