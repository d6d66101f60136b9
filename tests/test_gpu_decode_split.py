"""Both ways the M <= 16 INT4 kernel can share a tile's K range between thread blocks --
the stream-K grid (partial tiles through the workspace) and thread-block clusters (partial
tiles through distributed shared memory) -- against the CPU oracle, through the C ABI.

Bars: bf16 outputs within max-abs <= 1e-2 * ||y_ref||_inf and mean relative error <= 2e-3;
one-hot activations reproduce the dequantised weights bit for bit; repeated calls are
bit-identical (both reductions add in a fixed order).
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


@pytest.fixture(params=["stream_k", "cluster"])
def split(request, capi):
    capi.set_option(capi.OPT_DECODE_SPLIT, capi.SPLIT_STREAM_K if request.param == "stream_k" else capi.SPLIT_CLUSTER)
    yield request.param
    capi.set_option(capi.OPT_DECODE_SPLIT, capi.SPLIT_AUTO)


def make_ctx(capi, layer, flags=0, hint=0):
    qw, s, z, b = to_device_layer(layer, "cuda")
    return capi.WoqContext(qw, s, z, b, layer["n"], layer["k"], capi.DTYPE_INT4, layer["g"],
                           capi.LOWP_BF16, layout_flags=flags | capi.LAYOUT_STREAM_ONLY, kernel_hint=hint)


def oracle_y(layer, x, fusion=O.FUSE_NONE, others=()):
    return O.woq_linear_bf16(x, layer["qw"], layer["s16"], layer["z"], layer["bias"],
                             O.WOQ_DTYPE_INT4, layer["g"], fusion, others)


def assert_parity(y, y_ref):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL, f"max-abs/inf-norm {mx:.3e}"
    assert mr <= O.MEAN_REL_TOL, f"mean rel {mr:.3e}"


# (N, K, G): tiles x k-blocks chosen so that the cluster grid takes 1, 2, 3, 4, 5 and 8 CTAs per
# tile on a 148-SM part, with slices that do and do not divide evenly
SHAPES = [(4096, 4096, 128), (6144, 4096, 128), (1280, 8192, 128), (8192, 1024, 128), (3584, 2560, 128),
          (9472, 1024, 64), (2368, 3072, -1), (200, 4096, 128), (16384, 512, 128)]


@pytest.mark.parametrize("m", [1, 5, 8, 16])
@pytest.mark.parametrize("n,k,g", SHAPES)
def test_parity_in_both_splits(capi, split, n, k, g, m):
    layer = make_int4_layer(n, k, g, seed=n + k + m, bias=(n % 128 != 0))
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=m)
    xg = bf16_tensor(x, "cuda")
    y0 = ctx.linear(xg)
    y = bf16_numpy(y0)
    ctx.workspace(m).status()
    assert_parity(y, oracle_y(layer, x))
    for _ in range(3):
        assert torch.equal(ctx.linear(xg), y0)


@pytest.mark.parametrize("m", [1, 16])
@pytest.mark.parametrize("n,k,g", [(4096, 4096, 128), (1280, 8192, 128), (6144, 4096, 128)])
def test_scale_after_sum_in_both_splits(capi, split, n, k, g, m):
    layer = make_int4_layer(n, k, g, seed=n + 3 * m)
    ctx = make_ctx(capi, layer, hint=capi.HINT_STREAM_FAST)
    x = make_acts(m, k, seed=m + 100)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    assert_parity(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [1, 7, 16])
def test_one_hot_rows_are_the_dequantised_weights(capi, split, m):
    n, k, g = 2048, 4096, 128
    layer = make_int4_layer(n, k, g, seed=11 + m)
    ctx = make_ctx(capi, layer)
    w_ref = O.dequantize_weight(layer["qw"], layer["s16"], layer["z"], O.WOQ_DTYPE_INT4, k, g)
    rng = np.random.default_rng(m)
    for _ in range(4):
        cols = rng.choice(k, size=m, replace=False)
        x = np.zeros((m, k), np.float32)
        x[np.arange(m), cols] = 1.0
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
        np.testing.assert_array_equal(y.view(np.uint32), w_ref[:, cols].T.copy().view(np.uint32))
    ctx.workspace(m).status()


FUSIONS = [(O.FUSE_GELU_TANH, 0), (O.FUSE_SILU, 0), (O.FUSE_ADD, 1), (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1)]


@pytest.mark.parametrize("fusion,n_others", FUSIONS)
@pytest.mark.parametrize("m", [2, 16])
def test_fused_post_ops_in_both_splits(capi, split, fusion, n_others, m):
    n, k = 1664, 4096
    layer = make_int4_layer(n, k, 128, seed=fusion + 11, std=0.05, bias=True)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=fusion)
    others = [make_acts(m, n, seed=50 + i) for i in range(n_others)]
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), fusion, [bf16_tensor(o, "cuda") for o in others]))
    ctx.workspace(m).status()
    assert_parity(y, oracle_y(layer, x, fusion, others))


@pytest.mark.parametrize("m", [1, 9])
def test_gate_up_silu_mul_in_both_splits(capi, split, m):
    inter, k = 3584, 4096
    layer = make_int4_layer(2 * inter, k, 128, seed=77, std=0.05)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_GATE_UP)
    x = make_acts(m, k, seed=m + 5)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_SILU_MUL))
    ctx.workspace(m).status()
    assert y.shape == (m, inter)
    assert_parity(y, oracle_y(layer, x, O.FUSE_SILU_MUL))


def test_many_calls_back_to_back_in_a_graph(capi, split):
    """Programmatic dependent launch lets a launch start before the previous one has ended;
    a chain of calls that feed each other must still see finished inputs."""
    n = k = 2048
    layers = [make_int4_layer(n, k, 128, seed=300 + i, std=0.03) for i in range(4)]
    ctxs = [make_ctx(capi, L) for L in layers]
    x = make_acts(3, k, seed=1)
    bufs = [bf16_tensor(x, "cuda")] + [torch.empty((3, n), dtype=torch.bfloat16, device="cuda") for _ in ctxs]
    ws = capi.Workspace(ctxs[0].workspace_bytes(3), "cuda")

    def chain():
        for i, c in enumerate(ctxs):
            c.linear(bufs[i], capi.FUSE_RELU, out=bufs[i + 1], workspace=ws)

    chain()
    torch.cuda.synchronize()
    eager = bufs[-1].clone()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            chain()
    for _ in range(5):
        bufs[-1].zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(bufs[-1], eager)
    ws.status()
    ref = x
    for L in layers:
        ref = oracle_y(L, ref, O.FUSE_RELU)
    assert_parity(bf16_numpy(eager), ref)
