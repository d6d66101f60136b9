"""GPU parity of the tcgen05 INT4 kernel (exact bf16 tile dequantisation, fp32 accumulation
in TMEM) against the CPU oracle, for decode-size and prefill-size token counts."""
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


def make_ctx(capi, layer, flags=0):
    qw, s, z, b = to_device_layer(layer, "cuda")
    return capi.WoqContext(qw, s, z, b, layer["n"], layer["k"], capi.DTYPE_INT4, layer["g"],
                           capi.LOWP_BF16, layout_flags=flags, kernel_hint=capi.HINT_TENSOR_CORE)


def oracle_y(layer, x, fusion=O.FUSE_NONE, others=()):
    return O.woq_linear_bf16(x, layer["qw"], layer["s16"], layer["z"], layer["bias"],
                             O.WOQ_DTYPE_INT4, layer["g"], fusion, others)


def check(y, y_ref, tight=True):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)
    if tight:
        # same bf16 weights and fp32 accumulation as the oracle: only the summation order
        # differs, so almost every output is bit-identical
        assert (y == y_ref).mean() > 0.97, (y == y_ref).mean()
        assert mr < 2e-4, mr


@pytest.mark.parametrize("m", [1, 4, 16, 32, 100, 256, 300])
def test_small_layer(capi, m):
    layer = make_int4_layer(256, 512, 128, seed=10 + m)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, 512, seed=m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    check(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [1, 4, 32, 256])
def test_config1_single_linear(capi, m):
    layer = make_int4_layer(4096, 4096, 128, seed=1000)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, 4096, seed=1000 + m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    check(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [24, 64, 128, 256])
def test_many_pipeline_stages_per_cta(capi, m):
    """A long K and few tiles give every CTA dozens of pipeline stages, several tile segments and
    partial tiles at both ends: every shared-memory slot and every TMEM operand group is
    reused many times (mbarrier phases wrap)."""
    layer = make_int4_layer(1152, 16384, 128, seed=4242)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_TC_ONLY)
    x = make_acts(m, 16384, seed=m)
    for _ in range(2):
        y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    check(y, oracle_y(layer, x))


@pytest.mark.parametrize("m", [2, 17, 64, 129])
@pytest.mark.parametrize("n,k,g", [(64, 64, 64), (200, 320, 64), (768, 1536, 128), (96, 3584, 128),
                                   (1280, 1024, -1), (320, 2048, 512)])
def test_shapes(capi, m, n, k, g):
    layer = make_int4_layer(n, k, g, seed=n * 3 + k + m, bias=(n % 128 != 0))
    ctx = make_ctx(capi, layer)
    x = make_acts(m, k, seed=m)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda")))
    ctx.workspace(m).status()
    check(y, oracle_y(layer, x))


FUSIONS = [(O.FUSE_GELU_ERF, 0), (O.FUSE_GELU_TANH, 0), (O.FUSE_RELU, 0), (O.FUSE_SILU, 0),
           (O.FUSE_ADD, 1), (O.FUSE_ADD_ADD, 2), (O.FUSE_MUL, 1)]


@pytest.mark.parametrize("fusion,n_others", FUSIONS)
@pytest.mark.parametrize("m", [4, 63])
def test_fused_post_ops(capi, fusion, n_others, m):
    layer = make_int4_layer(640, 1024, 128, seed=fusion + 11, std=0.05, bias=True)
    ctx = make_ctx(capi, layer)
    x = make_acts(m, 1024, seed=fusion)
    others = [make_acts(m, 640, seed=50 + i) for i in range(n_others)]
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), fusion, [bf16_tensor(o, "cuda") for o in others]))
    check(y, oracle_y(layer, x, fusion, others), tight=False)


@pytest.mark.parametrize("m", [1, 7, 16, 200])
def test_gate_up_silu_mul(capi, m):
    inter, k = 1792, 1024
    layer = make_int4_layer(2 * inter, k, 128, seed=77, std=0.05)
    ctx = make_ctx(capi, layer, flags=capi.LAYOUT_GATE_UP)
    x = make_acts(m, k, seed=m + 5)
    y = bf16_numpy(ctx.linear(bf16_tensor(x, "cuda"), capi.FUSE_SILU_MUL))
    assert y.shape == (m, inter)
    check(y, oracle_y(layer, x, O.FUSE_SILU_MUL), tight=False)


def test_dump_matches_for_both_layouts(capi):
    layer = make_int4_layer(300, 512, 128, seed=3)
    ctx = make_ctx(capi, layer)
    w = bf16_numpy(ctx.dump_dequant())
    w_ref = O.dequantize_weight(layer["qw"], layer["s16"], layer["z"], O.WOQ_DTYPE_INT4, 512, 128)
    np.testing.assert_array_equal(w.view(np.uint32), w_ref.view(np.uint32))


def test_repeatable(capi):
    layer = make_int4_layer(4096, 4096, 128, seed=5)
    ctx = make_ctx(capi, layer)
    x = bf16_tensor(make_acts(48, 4096, seed=9), "cuda")
    y0 = ctx.linear(x).clone()
    for _ in range(3):
        assert torch.equal(ctx.linear(x), y0)


def test_many_full_width_launches_in_a_row(capi):
    """Several hundred 256-token launches on two weight copies with nothing between them: every
    one completes (the status word stays clear) and gives the bits of the first."""
    layers = [make_int4_layer(8192, 4096, 128, seed=70 + i) for i in range(2)]
    ctxs = [make_ctx(capi, layer) for layer in layers]
    x = bf16_tensor(make_acts(256, 4096, seed=3), "cuda")
    ws = capi.Workspace(ctxs[0].workspace_bytes(256), "cuda")
    outs = [torch.empty((256, 8192), dtype=torch.bfloat16, device="cuda") for _ in ctxs]
    want = []
    for c, out in zip(ctxs, outs):
        c.linear(x, out=out, workspace=ws)
        want.append(out.clone())
    for _ in range(200):
        for c, out in zip(ctxs, outs):
            c.linear(x, out=out, workspace=ws)
    torch.cuda.synchronize()
    ws.status()
    for out, w in zip(outs, want):
        assert torch.equal(out, w)


@pytest.mark.parametrize("m", [24, 200])
def test_launches_back_to_back(capi, m):
    """A chain in which every linear reads the previous one's output and all share one workspace,
    launched without host synchronisation and as a CUDA graph: same bits as the chain with a
    synchronisation after every launch."""
    dims = [(1024, 512), (768, 1024), (512, 768), (1024, 512)]
    layers = [make_int4_layer(n, k, 128, seed=900 + i, std=0.05) for i, (n, k) in enumerate(dims)]
    ctxs = [make_ctx(capi, layer) for layer in layers]
    ws = capi.Workspace(max(c.workspace_bytes(m) for c in ctxs), "cuda")
    x = bf16_tensor(make_acts(m, 512, seed=m), "cuda")
    bufs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for n, _ in dims]

    def chain(sync):
        h = x
        for c, out in zip(ctxs, bufs):
            c.linear(h, out=out, workspace=ws)
            if sync:
                torch.cuda.synchronize()
            h = out
        return h

    want = chain(True).clone()
    for _ in range(5):
        got = chain(False)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        chain(False)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(3):
                chain(False)
        for _ in range(4):
            graph.replay()
        stream.synchronize()
    assert torch.equal(bufs[-1], want)
    ws.status()
