"""The reference-facing Python surface on the GPU: WeightOnlyQuantizedLinear and friends call
torch.ops.torch_ipex.* (CUDA dispatch), which run the sm_100a kernels.  Modelled on the
reference's own WOQ unit tests (tests/cpu/test_quantization_default_recipe.py,
tests/cpu/test_ipex_llm_quantization.py)."""
import copy
import io
import os

import numpy as np
import pytest
import torch
from torch import nn

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


def parity(y, y_ref):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)


def make_linear(n, k, bias, seed):
    torch.manual_seed(seed)
    lin = nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    return lin


def oracle_from_linear(lin, x, group, fusion=O.FUSE_NONE, others=()):
    """Oracle output for the codes the module itself produces: the weight is quantised by the
    package's quantiser on the GPU, as from_float does (its CPU results are pinned against the
    reference's golden outputs; a GPU division can differ from the CPU one in the last bit, which
    moves about one code in 10^5), then the oracle does the linear."""
    from ipex_b200 import quantization as q

    w = lin.weight.detach().float().cuda()
    if group > 0:
        qw, s, z = q.quantize_per_block(w, q.WoqWeightDtype.INT4, group)
    else:
        qw, s, z = q.quantize_per_channel(w, q.WoqWeightDtype.INT4)
    qw, s, z = qw.cpu().numpy(), s.cpu().numpy(), z.cpu().numpy()
    b = None if lin.bias is None else lin.bias.detach().float().numpy()
    return O.woq_linear_bf16(x, qw, s, z, b, O.WOQ_DTYPE_INT4, group, fusion, others), (qw, s, z)


@pytest.mark.parametrize("m", [4, 100])
@pytest.mark.parametrize("group", [128, -1])
def test_from_float_int4_bf16(ipex, m, group):
    q = ipex.quantization
    lin = make_linear(500, 1024, True, seed=group + m)  # N = 500 is padded inside
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=group).global_qconfig
    ref_lin = copy.deepcopy(lin)
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    x = make_acts(m, 1024, seed=m)
    y = mod(bf16_tensor(x, "cuda"))
    assert y.shape == (m, 500) and y.dtype == torch.bfloat16
    y_ref, (qw, s, z) = oracle_from_linear(ref_lin, x, group)
    parity(bf16_numpy(y), y_ref)
    # the module's weight attribute is the plain quantised weight: bit-exact round trip
    np.testing.assert_array_equal(mod.weight.cpu().numpy(), qw)
    np.testing.assert_array_equal(mod._op_context.get_weight().cpu().numpy(), qw)
    assert "dtype=int4" in mod.extra_repr() and f"group_size={group}" in mod.extra_repr()
    # leading dimensions are kept
    y3 = mod(bf16_tensor(x, "cuda").reshape(2, m // 2, 1024))
    assert y3.shape == (2, m // 2, 500)
    assert torch.equal(y3.reshape(m, 500), y)


def test_op_without_context_matches_module(ipex):
    q = ipex.quantization
    lin = make_linear(256, 512, False, seed=1)
    w = lin.weight.detach().cuda()
    qw, s, z = q.quantize_per_block(w, q.WoqWeightDtype.INT4, 128)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=128).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    x = torch.randn(7, 512, device="cuda").bfloat16()
    y1 = mod(x)
    y2 = torch.ops.torch_ipex.woq_linear(x, qw, "int4", [256, 512], [s], [z], None, None, 128, 2, -1, None)
    assert torch.equal(y1, y2)
    # the reference's pack op feeds the same context-free form
    pw, ps, pz, pb, pg = torch.ops.ipex_prepack.woq_linear_pack_weight(qw, "int4", [256, 512], s, z, None, None, 128, 2)
    assert [t.dtype for t in ps] == [torch.float32, torch.float16, torch.bfloat16] and pb is None and pg is None
    y3 = torch.ops.torch_ipex.woq_linear(x, pw, "int4", [256, 512], ps, pz, pb, pg, 128, 2, -1, None)
    assert torch.equal(y1, y3)
    assert torch.equal(torch.ops.ipex_prepack.woq_linear_unpack_weight(pw, "int4", [256, 512], 2), qw)


def test_fused_epilogue_modules(ipex):
    from ipex_b200.transformers.fusions import linear_fusion as F

    q = ipex.quantization
    qc = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=128).global_qconfig
    inter, hidden, m = 1792, 1024, 6
    gate, up = make_linear(inter, hidden, False, 2), make_linear(inter, hidden, False, 3)
    down = make_linear(hidden, inter, False, 4)
    refs = [copy.deepcopy(t) for t in (gate, up, down)]
    for t in (gate, up, down):
        t.qconfig = qc
    W = ipex.nn.modules.WeightOnlyQuantizedLinear
    qg, qu, qd = W.from_float(gate), W.from_float(up), W.from_float(down)
    x = make_acts(m, hidden, seed=5)
    xg = bf16_tensor(x, "cuda")
    # silu(gate) * up, the reference's two-op composition
    y = F._IPEXlinearSiluMulCPU(qg, qu, woq=True)(xg)
    g_ref, (qwg, sg, zg) = oracle_from_linear(refs[0], x, 128, O.FUSE_SILU)
    y_ref, (qwu, su, zu) = oracle_from_linear(refs[1], x, 128, O.FUSE_MUL, [g_ref])
    parity(bf16_numpy(y), y_ref)
    # the single-kernel version of the same thing on the stacked weight
    fused = F._IPEXlinearFusedGateUp.from_quantized(
        torch.from_numpy(np.concatenate([qwg, qwu])).cuda(), q.WoqWeightDtype.INT4, [2 * inter, hidden],
        torch.from_numpy(np.concatenate([sg, su])).cuda(), torch.from_numpy(np.concatenate([zg, zu])).cuda(),
        128, q.WoqLowpMode.BF16)
    parity(bf16_numpy(fused(xg)), y_ref)
    # linear + residual add
    r = make_acts(m, hidden, seed=6)
    a = bf16_numpy(y)
    z_ = F._IPEXlinearAddCPU(qd, woq=True)(y, bf16_tensor(r, "cuda"))
    z_ref, _ = oracle_from_linear(refs[2], a, 128, O.FUSE_ADD, [r])
    parity(bf16_numpy(z_), z_ref)
    for cls, fusion in ((F._IPEXlinearGeluCPU, O.FUSE_GELU_ERF), (F._IPEXlinearNewGeluCPU, O.FUSE_GELU_TANH),
                        (F._IPEXlinearReluCPU, O.FUSE_RELU), (F._IPEXlinearSiluCPU, O.FUSE_SILU)):
        out = cls(qd, woq=True)(y)
        ref, _ = oracle_from_linear(refs[2], a, 128, fusion)
        parity(bf16_numpy(out), ref)


def test_awq_checkpoint_through_from_weight(ipex, golden_dir):
    """reference: tests/cpu/test_ipex_llm_quantization.py:113-151 (same tensors, same tolerance)"""
    f = np.load(os.path.join(golden_dir, "awq_fixture.npz"))
    from ipex_b200.llm.quantization import IPEXWeightOnlyQuantizedLinear, QuantDtype, QuantMethod

    qweight = torch.from_numpy(f["qweight"])
    qzeros = torch.from_numpy(f["qzeros"])
    scales = torch.from_numpy(O.from_bf16_bits(f["scales_bf16"])).bfloat16()
    bias = torch.from_numpy(O.from_bf16_bits(f["bias_bf16"])).bfloat16()
    k, n = qweight.shape[0], qweight.shape[1] * 8
    mod = IPEXWeightOnlyQuantizedLinear.from_weight(qweight, scales, qzeros, k, n, None, bias, 128, None,
                                                    QuantMethod.AWQ_GEMM, QuantDtype.INT4)
    x = O.from_bf16_bits(f["act_bf16"])
    y = bf16_numpy(mod(bf16_tensor(x, "cuda")))
    assert np.abs(y - O.from_bf16_bits(f["y_ref_bf16"])).max() <= 0.1


def test_gptq_checkpoint_layout(ipex):
    from ipex_b200.llm.quantization import IPEXWeightOnlyQuantizedLinear, QuantMethod

    n, k, g = 256, 512, 128
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    qw, s, z = O.quantize_per_block(w, O.WOQ_DTYPE_INT4, g)
    q = O.unpack_nibbles(qw).astype(np.uint32)  # [N, K]
    # GPTQ: qweight [K/8, N] int32 (nibble j of word r = k 8r+j), qzeros [groups, N/8] stored minus one
    qT = q.T.reshape(k // 8, 8, n)
    gq = np.zeros((k // 8, n), dtype=np.uint32)
    for j in range(8):
        gq |= qT[:, j, :] << (4 * j)
    zz = (z.T.astype(np.int64) - 1) % 16  # [groups, N]
    gz = np.zeros((k // g, n // 8), dtype=np.uint32)
    for j in range(8):
        gz |= zz[:, j::8].astype(np.uint32) << (4 * j)
    mod = IPEXWeightOnlyQuantizedLinear.from_weight(
        torch.from_numpy(gq.view(np.int32)), torch.from_numpy(s.T.copy()).half(),
        torch.from_numpy(gz.view(np.int32)), k, n, None, None, g, None, QuantMethod.GPTQ_GEMM)
    np.testing.assert_array_equal(mod.weight.cpu().numpy(), qw)
    x = make_acts(5, k, seed=2)
    y = bf16_numpy(mod(bf16_tensor(x, "cuda")))
    parity(y, O.woq_linear_bf16(x, qw, s.astype(np.float16), z, None, O.WOQ_DTYPE_INT4, g))


def test_gptq_act_order_g_idx(ipex):
    """GPTQ act-order: group membership of the input channels given by g_idx (a shuffled
    assignment), through the checkpoint entry point and through the plain prepack op; the
    context hands back the unshuffled weight and survives pickling."""
    from ipex_b200.llm.quantization import IPEXWeightOnlyQuantizedLinear, QuantMethod

    n, k, g = 192, 512, 128
    rng = np.random.default_rng(3)
    g_idx = rng.permutation(np.arange(k) // g).astype(np.int32)
    q = rng.integers(0, 16, (n, k)).astype(np.uint32)
    qw = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    s = (rng.random((n, k // g)) * 0.01 + 0.002).astype(np.float16)
    z = rng.integers(1, 16, (n, k // g)).astype(np.float32)
    x = make_acts(6, k, seed=4)
    y_ref = O.woq_linear_bf16_act_order(x, qw, s, z, None, g_idx)

    # plain prepack op
    ctx = torch.ops.ipex_prepack.weight_only_qlinear_prepack(
        torch.from_numpy(qw).cuda(), 2, [n, k], torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(), None,
        torch.from_numpy(g_idx).cuda(), None, g, 2, -1)
    y = torch.ops.torch_ipex.ipex_woq_linear(bf16_tensor(x, "cuda"), ctx.get_data_handle())
    parity(bf16_numpy(y), y_ref)
    np.testing.assert_array_equal(ctx.get_weight().cpu().numpy(), qw)
    np.testing.assert_array_equal(ctx.get_g_idx().cpu().numpy(), g_idx)
    buf = io.BytesIO()
    torch.save(ctx, buf)
    buf.seek(0)
    ctx2 = torch.load(buf, weights_only=False)
    y2 = torch.ops.torch_ipex.ipex_woq_linear(bf16_tensor(x, "cuda"), ctx2.get_data_handle())
    assert torch.equal(y, y2)

    # AutoGPTQ checkpoint tensors
    qT = q.T.reshape(k // 8, 8, n)
    gq = np.zeros((k // 8, n), dtype=np.uint32)
    for j in range(8):
        gq |= qT[:, j, :] << (4 * j)
    zz = (z.T.astype(np.int64) - 1) % 16
    gz = np.zeros((k // g, n // 8), dtype=np.uint32)
    for j in range(8):
        gz |= zz[:, j::8].astype(np.uint32) << (4 * j)
    mod = IPEXWeightOnlyQuantizedLinear.from_weight(
        torch.from_numpy(gq.view(np.int32)), torch.from_numpy(s.T.copy()), torch.from_numpy(gz.view(np.int32)),
        k, n, None, None, g, torch.from_numpy(g_idx), QuantMethod.GPTQ_GEMM)
    y3 = mod(bf16_tensor(x, "cuda"))
    assert torch.equal(y3, y)


@pytest.mark.parametrize("act_mode", ["PER_BATCH_SYM", "PER_BATCH", "PER_TENSOR_SYM", "PER_TENSOR"])
def test_int8_lowp_module(ipex, act_mode):
    q = ipex.quantization
    lin = make_linear(384, 1024, True, seed=9)
    ref = copy.deepcopy(lin)
    mode = getattr(q.WoqActQuantMode, act_mode)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT8, lowp_mode=q.WoqLowpMode.INT8, act_quant_mode=mode).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    x = O.rne_bf16(make_acts(33, 1024, seed=3) + 0.2)
    y = bf16_numpy(mod(bf16_tensor(x, "cuda")))
    qw, s, _ = O.quantize_per_channel(ref.weight.detach().numpy(), O.WOQ_DTYPE_INT8, sym=True)
    parity(y, O.woq_linear_int8(x, qw, s, ref.bias.detach().numpy(), act_mode=int(mode)))


def test_op_context_pickles_in_plain_format(ipex):
    q = ipex.quantization
    lin = make_linear(128, 256, True, seed=11)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=64).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    x = torch.randn(3, 256, device="cuda").bfloat16()
    y = mod(x)
    buf = io.BytesIO()
    torch.save(mod._op_context, buf)
    buf.seek(0)
    ctx2 = torch.load(buf, weights_only=False)
    y2 = torch.ops.torch_ipex.ipex_woq_linear(x, ctx2.get_data_handle())
    assert torch.equal(y, y2)
    assert torch.equal(ctx2.get_weight(), mod._op_context.get_weight())


def test_autocast_and_errors(ipex):
    q = ipex.quantization
    lin = make_linear(128, 256, False, seed=12)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=128).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    x32 = torch.randn(4, 256, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = mod(x32)
    assert y.dtype == torch.bfloat16
    assert mod(x32).dtype == torch.float32          # without autocast the input dtype comes back
    with pytest.raises(RuntimeError, match="in_features"):
        mod(torch.randn(4, 128, device="cuda").bfloat16())
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(torch.randn(4, 256).bfloat16())


def test_llm_optimize_swaps_linears(ipex):
    q = ipex.quantization

    class MLP(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(256, 512, bias=False)
            self.down = nn.Linear(512, 256, bias=False)
            self.lm_head = nn.Linear(256, 100, bias=False)

        def forward(self, x):
            return self.lm_head(self.down(torch.relu(self.up(x))))

    torch.manual_seed(0)
    model = MLP()
    qmap = q.get_weight_only_quant_qconfig_mapping(weight_dtype=q.WoqWeightDtype.INT4,
                                                   lowp_mode=q.WoqLowpMode.BF16, group_size=128)
    opt = ipex.llm.optimize(model, dtype=torch.bfloat16, quantization_config=qmap)
    W = ipex.nn.modules.WeightOnlyQuantizedLinear
    assert isinstance(opt.up, W) and isinstance(opt.down, W) and isinstance(opt.lm_head, nn.Linear)
    x = torch.randn(5, 256, device="cuda").bfloat16()
    y = opt(x)
    y_ref = model.cuda().bfloat16()(x)
    assert torch.nn.functional.cosine_similarity(y.float().flatten(), y_ref.float().flatten(), dim=0) > 0.98


def test_row_parallel_shards_sum_to_the_full_layer(ipex):
    """Single-process simulation of the K-sharded tensor-parallel layer, like the reference's
    test_g_idx_tp (tests/cpu/test_quantization_default_recipe.py:1406-1520)."""
    q = ipex.quantization
    n, k, g, p = 256, 1024, 128, 2
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    qw, s, z = O.quantize_per_block(w, O.WOQ_DTYPE_INT4, g)
    x = make_acts(9, k, seed=1)
    xg = bf16_tensor(x, "cuda")
    ys = []
    for r in range(p):
        ks = k // p
        ctx = torch.ops.ipex_prepack.weight_only_qlinear_prepack(
            torch.from_numpy(qw[:, r * ks // 2:(r + 1) * ks // 2].copy()).cuda(), 2, [n, ks],
            torch.from_numpy(s[:, r * ks // g:(r + 1) * ks // g].copy()).half().cuda(),
            torch.from_numpy(z[:, r * ks // g:(r + 1) * ks // g].copy()).cuda(), None, None, None, g, 2, -1)
        ys.append(torch.ops.torch_ipex.ipex_woq_linear(xg[:, r * ks:(r + 1) * ks], ctx.get_data_handle()))
    y = bf16_numpy((ys[0].float() + ys[1].float()).bfloat16())
    shards = [qw[:, r * k // p // 2:(r + 1) * k // p // 2] for r in range(p)]
    y_ref = O.row_parallel_linear(x, shards, [s.astype(np.float16)[:, r * 4:(r + 1) * 4] for r in range(p)],
                                  [z[:, r * 4:(r + 1) * 4] for r in range(p)], None, O.WOQ_DTYPE_INT4, g)
    parity(y, y_ref)


def test_pickle_state_is_the_reference_twelve_tuple_and_load_from_ctx(ipex):
    q = ipex.quantization
    lin = make_linear(256, 512, True, seed=31)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=128).global_qconfig
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    state = mod._op_context.__getstate__()
    if len(state) != 12 and isinstance(state[0], tuple):  # some torch versions wrap the C++ state
        state = state[0]
    assert len(state) == 12, [type(v) for v in state]  # csrc/cpu/jit/cpu/kernels/OpContext.h:363-375
    other = make_linear(256, 512, True, seed=32)
    other.qconfig = lin.qconfig
    mod2 = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(other)
    x = torch.randn(5, 512, device="cuda").bfloat16()
    assert not torch.equal(mod(x), mod2(x))
    mod2._op_context.load_from_ctx(mod._op_context)
    assert torch.equal(mod(x), mod2(x))
    assert torch.equal(mod2._op_context.get_weight(), mod._op_context.get_weight())


def test_second_tiling_is_packed_on_first_large_batch(ipex):
    """A context made through the ops keeps the streaming tiling; the tensor-core tiling appears
    with the first call of more than 16 tokens and gives the same numbers as a context that had
    it from the start (through the C ABI)."""
    q = ipex.quantization
    capi = ipex._capi
    lin = make_linear(384, 1024, False, seed=41)
    lin.qconfig = q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16, group_size=128).global_qconfig
    w = lin.weight.detach().float().cuda()
    mod = ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)
    qw, s, z = q.quantize_per_block(w, q.WoqWeightDtype.INT4, 128)
    both = capi.WoqContext(qw, s, z, None, 384, 1024, capi.DTYPE_INT4, 128, capi.LOWP_BF16)
    small = torch.randn(8, 1024, device="cuda").bfloat16()
    large = torch.randn(200, 1024, device="cuda").bfloat16()
    assert torch.equal(mod(small), both.linear(small))
    assert torch.equal(mod(large), both.linear(large))
    assert torch.equal(mod(small), both.linear(small))
    torch.ops.torch_ipex.woq_check_status()
