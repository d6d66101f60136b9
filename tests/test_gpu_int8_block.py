"""INT8 compute with K-block scaling (woq_int8_block.cu): INT4 or INT8 weights, every activation
quantisation mode of the reference, against the CPU oracle through the C ABI.

Bars: activation codes, scales, zero points and the int32 block accumulators bit-exact; bf16
outputs within max-abs <= 1e-2 * ||y_ref||_inf and mean relative error <= 2e-3."""
import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, make_acts

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ipex():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ipex_b200

    ipex_b200.load_ops()
    return ipex_b200


def make_layer(kind, n, k, g, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    dt = O.WOQ_DTYPE_INT4 if kind.startswith("int4") else O.WOQ_DTYPE_INT8
    sym = kind.endswith("_sym")
    if g > 0:
        qw, s, z = O.quantize_per_block(w, dt, g, sym)
    else:
        qw, s, z = O.quantize_per_channel(w, dt, sym)
        s = s[:, None]
        z = None if z is None else z[:, None]
    return qw, s, z, dt


def make_ctx(capi, qw, s, z, dt, n, k, g, mode, bias=None):
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    return capi.WoqContext(t(qw), t(s), t(z), t(bias), n, k, dt, g, capi.LOWP_INT8, act_quant_mode=mode)


def parity(y, ref):
    mx, mr = O.parity_metrics(y, ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


LAYERS = [("int4", 96, 512, 128), ("int4", 200, 1024, 64), ("int4_sym", 64, 384, 128), ("int4", 80, 640, -1),
          ("int8_sym", 112, 512, -1), ("int8", 64, 256, 128)]


@pytest.mark.parametrize("mode", range(8))
@pytest.mark.parametrize("kind,n,k,g", LAYERS)
def test_internals_bit_exact_and_outputs(ipex, kind, n, k, g, mode):
    capi = ipex._capi
    if kind == "int8_sym" and g <= 0 and mode in (0, 2, 4, 6):
        pytest.skip("whole-K activation ranges on per-channel INT8 weights belong to the tcgen05 INT8 kernel")
    qw, s, z, dt = make_layer(kind, n, k, g, seed=n + k)
    rng = np.random.default_rng(mode)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float32) if mode % 2 else None
    ctx = make_ctx(capi, qw, s, z, dt, n, k, g, mode, bias)
    assert ctx.route() == capi.ROUTE_INT8_BLOCK
    for m in (1, 5, 8, 19, 70):  # up to 16 tokens the 16 x 8 kernel, above it the 64 x 64 one
        x = O.rne_bf16(make_acts(m, k, seed=m + mode) + (0.0 if mode >= 4 else 0.31))
        if m > 2:
            x[1, : O.int8_block_k(k, g)] = 0.0  # a block of zeros: scale 0, codes 0
        y_ref, blocks, qa_ref, sa_ref, zpa_ref = O.woq_linear_int8_blocks(x, qw, dt, s, z, bias, g, mode,
                                                                          return_blocks=True)
        qa, sa, zpa, acc = ctx.int8_block_internals(bf16_tensor(x, "cuda"))
        ctx.workspace(m).status()
        np.testing.assert_array_equal(qa.cpu().numpy(), qa_ref.view(np.uint8))
        np.testing.assert_array_equal(sa.cpu().numpy(), sa_ref)
        if zpa_ref is None:
            assert not zpa.any()
        else:
            np.testing.assert_array_equal(zpa.cpu().numpy(), zpa_ref)
        np.testing.assert_array_equal(acc.cpu().numpy(), blocks)
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
        parity(y, y_ref)


@pytest.mark.parametrize("fusion,n_others", [(O.FUSE_GELU_TANH, 0), (O.FUSE_SILU, 0), (O.FUSE_ADD, 1),
                                             (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1)])
def test_post_ops(ipex, fusion, n_others):
    capi = ipex._capi
    n, k, g = 160, 512, 128
    qw, s, z, dt = make_layer("int4", n, k, g, seed=fusion)
    ctx = make_ctx(capi, qw, s, z, dt, n, k, g, 7)
    for m in (11, 90):  # both kernels of the route
        x = make_acts(m, k, seed=fusion + 1)
        others = [make_acts(m, n, seed=30 + i) for i in range(n_others)]
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), fusion, [bf16_tensor(o, "cuda") for o in others]))
        parity(y, O.woq_linear_int8_blocks(x, qw, dt, s, z, None, g, 7, fusion, others))


def test_llama_sized_layer_decode_and_prefill_tokens(ipex):
    """QKV of Llama-3-8B (6144 x 4096), INT4 g128 weights, INT8 compute, the reference's default
    activation mode (per token and K block, symmetric); the oracle on a subset of the rows."""
    capi = ipex._capi
    n, k, g = 6144, 4096, 128
    qw, s, z, dt = make_layer("int4", n, k, g, seed=1)
    ctx = make_ctx(capi, qw, s, z, dt, n, k, g, 7)
    rows = np.arange(0, n, 13)
    for m in (1, 8, 64, 300):
        x = make_acts(m, k, seed=m)
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))[:, rows]
        ctx.workspace(m).status()
        parity(y, O.woq_linear_int8_blocks(x, qw[rows], dt, s[rows], z[rows], None, g, 7))


def test_default_int8_lowp_recipes_through_the_module(ipex):
    """lowp_mode INT8 with the reference's default act_quant_mode (PER_BATCH_IC_BLOCK_SYM = 7,
    quantization/_qconfig.py:189-307), for INT4 and for INT8 weights."""
    q = ipex.quantization
    for wd, dt, g in ((q.WoqWeightDtype.INT4, O.WOQ_DTYPE_INT4, 128), (q.WoqWeightDtype.INT8, O.WOQ_DTYPE_INT8, -1)):
        torch.manual_seed(3)
        lin = torch.nn.Linear(512, 192, bias=True)
        with torch.no_grad():
            lin.weight.mul_(0.02 / lin.weight.std())
        w = lin.weight.detach().float().numpy().copy()
        b = lin.bias.detach().float().numpy().copy()
        cfg = q.get_weight_only_quant_qconfig_mapping(weight_dtype=wd, lowp_mode=q.WoqLowpMode.INT8, group_size=g)
        assert cfg.global_qconfig.act_quant_mode == 7
        lin.qconfig = cfg.global_qconfig
        mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
        sym = wd == q.WoqWeightDtype.INT8
        if g > 0:
            qw, s, z = O.quantize_per_block(w, dt, g, sym)
        else:
            qw, s, z = O.quantize_per_channel(w, dt, sym)
            s, z = s[:, None], (None if z is None else z[:, None])
        x = make_acts(6, 512, seed=4)
        y = bf16_numpy(mod(bf16_tensor(x, "cuda")))
        parity(y, O.woq_linear_int8_blocks(x, qw, dt, s, z, b, g, 7))
