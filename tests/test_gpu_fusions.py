"""Linears fused across modules (concatenated q/k/v, gate/up in one kernel) and the
low-precision checkpoint loader, on the GPU through the Python surface.  Modelled on the
reference's tests/cpu/test_ipex_optimize_transformers.py (fused modules against the unfused
model) and tests/cpu/test_quantization_default_recipe.py (low-precision checkpoints)."""
import copy

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


def qmap(ipex, lowp="BF16", group=128, act="PER_BATCH_IC_BLOCK_SYM"):
    q = ipex.quantization
    return q.get_weight_only_quant_qconfig_mapping(
        weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=getattr(q.WoqLowpMode, lowp), group_size=group,
        act_quant_mode=getattr(q.WoqActQuantMode, act))


def woq(ipex, lin, qm):
    lin = copy.deepcopy(lin)
    lin.qconfig = qm.global_qconfig
    return ipex.nn.modules.WeightOnlyQuantizedLinear.from_float(lin)


def oracle_of(mod, x, fusion=O.FUSE_NONE, others=()):
    """Oracle output from the codes the module holds."""
    c = mod._op_context
    n = c.get_weight_shape()[0]
    z = c.get_zero_points()
    b = c.get_bias()
    return O.woq_linear_bf16(
        x, c.get_weight().cpu().numpy(), c.get_scales().float().cpu().numpy().reshape(n, -1),
        None if z is None else z.float().cpu().numpy().reshape(n, -1),
        None if b is None else b.float().cpu().numpy(), O.WOQ_DTYPE_INT4, mod._group_size, fusion, others)


@pytest.mark.parametrize("m", [1, 7, 200])
@pytest.mark.parametrize("bias", [False, True])
def test_concat_qkv_equals_the_separate_linears(ipex, m, bias):
    """Grouped-query attention shapes: q 1024, k and v 256 out of K = 1024."""
    from ipex_b200.transformers.fusions.linear_fusion import _IPEXConcatLinear

    qm = qmap(ipex)
    mods = [woq(ipex, make_linear(n, 1024, bias, 10 + i), qm) for i, n in enumerate((1024, 256, 256))]
    holder = nn.Module()
    holder.linear_0, holder.linear_1, holder.linear_2, holder.num_concat = mods[0], mods[1], mods[2], 3
    cat = _IPEXConcatLinear(holder)
    assert cat.concat_linear is not None and cat.out_features == [1024, 256, 256]
    # the concatenated layer holds exactly the codes, scales and zero points of its parts
    c = cat.concat_linear._op_context
    assert torch.equal(c.get_weight(), torch.cat([mod._op_context.get_weight() for mod in mods], 0))
    assert torch.equal(c.get_scales().reshape(1536, -1),
                       torch.cat([mod._op_context.get_scales().reshape(mod.out_features, -1) for mod in mods], 0))
    x = make_acts(m, 1024, seed=m)
    xt = bf16_tensor(x, "cuda")
    y = cat(xt)
    assert y.shape == (m, 1536)
    parts = torch.cat([mod(xt) for mod in mods], -1)
    parity(bf16_numpy(y), oracle_of(cat.concat_linear, x))
    # against the three separate launches: same weights, fp32 partial sums may be grouped
    # differently when the tile count changes the K split
    d = (y.float() - parts.float()).abs().max().item()
    assert d <= 2.0 ** -7 * parts.float().abs().max().item(), d


def test_concat_falls_back_to_separate_outputs_for_act_order(ipex):
    from ipex_b200.transformers.fusions.linear_fusion import _IPEXConcatLinear

    n, k, g = 128, 256, 128
    rng = np.random.default_rng(5)
    mods = []
    for i in range(2):
        q = rng.integers(0, 16, (n, k)).astype(np.uint8)
        qw = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
        s = (rng.random((n, k // g)) * 0.01 + 0.002).astype(np.float16)
        z = rng.integers(1, 16, (n, k // g)).astype(np.float32)
        g_idx = rng.permutation(np.arange(k) // g).astype(np.int32)
        lin = nn.Linear(k, n, bias=False)
        lin.qconfig = qmap(ipex).global_qconfig
        mods.append(ipex.nn.modules.WeightOnlyQuantizedLinear.from_float_and_qweight(
            lin, torch.from_numpy(qw), ipex.quantization.WoqWeightDtype.INT4, torch.from_numpy(s),
            torch.from_numpy(z), None, group_size=g, g_idx=torch.from_numpy(g_idx)))
    holder = nn.Module()
    holder.linear_0, holder.linear_1, holder.num_concat = mods[0], mods[1], 2
    cat = _IPEXConcatLinear(holder)
    assert cat.concat_linear is None
    xt = bf16_tensor(make_acts(3, k, seed=1), "cuda")
    out = cat(xt)
    assert isinstance(out, tuple) and len(out) == 2
    assert torch.equal(out[0], mods[0](xt)) and torch.equal(out[1], mods[1](xt))


@pytest.mark.parametrize("m", [1, 16, 300])
def test_gate_up_from_two_linears(ipex, m):
    """_IPEXlinearFusedGateUp.from_linears(gate, up)(x) == silu(gate(x)) * up(x), the result the
    reference's _IPEXlinearSiluMul gives with two kernels."""
    from ipex_b200.transformers.fusions.linear_fusion import _IPEXlinearFusedGateUp, _IPEXlinearSiluMul

    qm = qmap(ipex)
    gate = woq(ipex, make_linear(768, 512, False, 1), qm)
    up = woq(ipex, make_linear(768, 512, False, 2), qm)
    fused = _IPEXlinearFusedGateUp.from_linears(gate, up)
    two = _IPEXlinearSiluMul(gate, up)
    x = make_acts(m, 512, seed=3 + m)
    xt = bf16_tensor(x, "cuda")
    y = fused(xt)
    assert y.shape == (m, 768)
    y2 = two(xt)
    d = (y.float() - y2.float()).abs().max().item()
    assert d <= 2.0 ** -6 * max(y2.float().abs().max().item(), 1e-6), d
    cg, cu = gate._op_context, up._op_context
    ref = O.woq_linear_bf16(
        x, torch.cat([cg.get_weight(), cu.get_weight()], 0).cpu().numpy(),
        torch.cat([cg.get_scales(), cu.get_scales()], 0).float().cpu().numpy().reshape(1536, -1),
        torch.cat([cg.get_zero_points(), cu.get_zero_points()], 0).float().cpu().numpy().reshape(1536, -1),
        None, O.WOQ_DTYPE_INT4, 128, O.FUSE_SILU_MUL)
    parity(bf16_numpy(y), ref)


class Attn(nn.Module):
    def __init__(self, hidden, heads, kv_heads):
        super().__init__()
        self.heads, self.kv_heads, self.hd = heads, kv_heads, hidden // heads
        self.q_proj = nn.Linear(hidden, heads * self.hd, bias=False)
        self.k_proj = nn.Linear(hidden, kv_heads * self.hd, bias=False)
        self.v_proj = nn.Linear(hidden, kv_heads * self.hd, bias=False)
        self.o_proj = nn.Linear(heads * self.hd, hidden, bias=False)

    def forward(self, x):
        b, t, _ = x.shape
        q = self.q_proj(x).view(b, t, self.heads, self.hd).transpose(1, 2)
        k = self.k_proj(x).view(b, t, self.kv_heads, self.hd).transpose(1, 2)
        v = self.v_proj(x).view(b, t, self.kv_heads, self.hd).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(o.transpose(1, 2).reshape(b, t, -1))


class Mlp(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)
        self.act_fn = nn.SiLU()

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, hidden=512, heads=8, kv_heads=2, inter=1024):
        super().__init__()
        self.self_attn = Attn(hidden, heads, kv_heads)
        self.mlp = Mlp(hidden, inter)
        self.n1 = nn.RMSNorm(hidden)
        self.n2 = nn.RMSNorm(hidden)
        self.lm_head = nn.Linear(hidden, 64, bias=False)

    def forward(self, x):
        x = x + self.self_attn(self.n1(x))
        x = x + self.mlp(self.n2(x))
        return self.lm_head(x)


@pytest.mark.parametrize("lowp", ["BF16", "INT8"])
def test_llm_optimize_fuses_llama_style_blocks(ipex, lowp):
    torch.manual_seed(0)
    model = Block()
    for p in model.parameters():
        if p.dim() == 2:
            with torch.no_grad():
                p.mul_(0.05 / p.std())
    qm = qmap(ipex, lowp)
    plain = ipex.llm.optimize(model, dtype=torch.bfloat16, quantization_config=qm, fuse=False)
    fused = ipex.llm.optimize(model, dtype=torch.bfloat16, quantization_config=qm)
    from ipex_b200.transformers.fusions.linear_fusion import _IPEXlinearFusedGateUp

    assert hasattr(fused.self_attn, "qkv_concat")
    if lowp == "BF16":
        assert isinstance(fused.mlp.gate_up_fused, _IPEXlinearFusedGateUp) and not hasattr(fused.mlp, "gate_proj")
    else:  # INT4 weights with INT8 compute take the K-block kernel, which has no gate/up layout
        assert hasattr(fused.mlp, "gate_proj") and not hasattr(fused.mlp, "gate_up_fused")
    assert isinstance(fused.lm_head, nn.Linear)
    for t in (1, 9):
        x = torch.randn(2, t, 512, device="cuda").bfloat16()
        a, b = fused(x).float(), plain(x).float()
        assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.999
        assert (a - b).abs().max() <= 0.03 * b.abs().max()
    # a second input through the same modules: the cached concatenated output must not be reused
    x2 = torch.randn(2, 9, 512, device="cuda").bfloat16()
    a, b = fused(x2).float(), plain(x2).float()
    assert (a - b).abs().max() <= 0.03 * b.abs().max()


# --------------------------------------------------------------------------------------------
# low-precision checkpoints


def _gptq_tensors(q, s, z, g):
    """[N, K] codes, [N, groups] scales / zero points -> AutoGPTQ qweight, scales, qzeros."""
    n, k = q.shape
    qT = q.T.astype(np.uint32).reshape(k // 8, 8, n)
    gq = np.zeros((k // 8, n), dtype=np.uint32)
    for j in range(8):
        gq |= qT[:, j, :] << (4 * j)
    zz = (z.T.astype(np.int64) - 1) % 16
    gz = np.zeros((k // g, n // 8), dtype=np.uint32)
    for j in range(8):
        gz |= zz[:, j::8].astype(np.uint32) << (4 * j)
    return (torch.from_numpy(gq.view(np.int32)), torch.from_numpy(s.T.copy()), torch.from_numpy(gz.view(np.int32)))


_AWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def _awq_pack(v):
    """[R, C] values 0..15 -> [R, C/8] int32 in AutoAWQ nibble order."""
    r, c = v.shape
    v = v.astype(np.uint32).reshape(r, c // 8, 8)
    out = np.zeros((r, c // 8), dtype=np.uint32)
    for j in range(8):
        out |= v[:, :, _AWQ_ORDER[j]] << (4 * j)
    return torch.from_numpy(out.view(np.int32))


class TwoLinears(nn.Module):
    def __init__(self, k, n, bias):
        super().__init__()
        self.fc1 = nn.Linear(k, n, bias=bias)
        self.norm = nn.LayerNorm(n)
        self.lm_head = nn.Linear(n, 32, bias=False)

    def forward(self, x):
        return self.lm_head(self.norm(self.fc1(x)))


def _checkpoint_case(seed, n=256, k=512, g=128):
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, (n, k)).astype(np.uint8)
    qw = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    s = (rng.random((n, k // g)) * 0.01 + 0.002).astype(np.float16)
    z = rng.integers(1, 16, (n, k // g)).astype(np.float32)
    bias = (rng.standard_normal(n) * 0.1).astype(np.float16)
    return q, qw, s, z, bias


@pytest.mark.parametrize("desc_act", [False, True])
def test_gptq_checkpoint_loader(ipex, desc_act):
    from ipex_b200.utils.weight_only_quantization import _convert_woq_with_low_precision_checkpoint

    n, k, g = 256, 512, 128
    q, qw, s, z, bias = _checkpoint_case(11)
    gq, gs, gz = _gptq_tensors(q, s, z, g)
    rng = np.random.default_rng(12)
    g_idx = rng.permutation(np.arange(k) // g).astype(np.int32) if desc_act else (np.arange(k) // g).astype(np.int32)
    head = torch.randn(32, n) * 0.05
    sd = {"fc1.qweight": gq, "fc1.scales": gs, "fc1.qzeros": gz, "fc1.g_idx": torch.from_numpy(g_idx),
          "fc1.bias": torch.from_numpy(bias), "lm_head.weight": head,
          "norm.weight": torch.full((n,), 1.5), "norm.bias": torch.full((n,), 0.25)}
    model = TwoLinears(k, n, True)
    out = _convert_woq_with_low_precision_checkpoint(
        model, qmap(ipex), sd, {"quant_method": "gptq", "desc_act": desc_act, "group_size": g})
    W = ipex.nn.modules.WeightOnlyQuantizedLinear
    assert isinstance(out.fc1, W) and isinstance(out.lm_head, nn.Linear)
    assert torch.equal(out.lm_head.weight.data, head) and torch.equal(out.norm.weight.data, sd["norm.weight"])
    np.testing.assert_array_equal(out.fc1._op_context.get_weight().cpu().numpy(), qw)
    assert (out.fc1._op_context.get_g_idx() is not None) == desc_act
    x = make_acts(5, k, seed=2)
    y = bf16_numpy(out.fc1(bf16_tensor(x, "cuda")))
    if desc_act:
        ref = O.woq_linear_bf16_act_order(x, qw, s, z, bias.astype(np.float32), g_idx)
    else:
        ref = O.woq_linear_bf16(x, qw, s, z, bias.astype(np.float32), O.WOQ_DTYPE_INT4, g)
    parity(y, ref)


def test_awq_checkpoint_loader_through_llm_optimize(ipex):
    n, k, g = 256, 512, 128
    q, qw, s, z, bias = _checkpoint_case(21)
    sd = {"fc1.qweight": _awq_pack(q.T), "fc1.scales": torch.from_numpy(s.T.copy()),
          "fc1.qzeros": _awq_pack(z.T.astype(np.uint8)), "fc1.bias": torch.from_numpy(bias),
          "lm_head.weight": torch.randn(32, n) * 0.05}
    model = TwoLinears(k, n, True)
    opt = ipex.llm.optimize(model, dtype=torch.bfloat16, quantization_config=qmap(ipex),
                            low_precision_checkpoint=(sd, {"quant_method": "awq"}))
    np.testing.assert_array_equal(opt.fc1._op_context.get_weight().cpu().numpy(), qw)
    assert opt.fc1._group_size == g
    x = make_acts(9, k, seed=4)
    y = bf16_numpy(opt.fc1(bf16_tensor(x, "cuda")))
    parity(y, O.woq_linear_bf16(x, qw, s, z, bias.astype(np.float32), O.WOQ_DTYPE_INT4, g))
    assert opt(bf16_tensor(x, "cuda")).shape == (9, 32)


@pytest.mark.parametrize("store", ["float8", "uint8"])
def test_fp8_block_scaled_checkpoint_loader(ipex, store):
    """DeepSeek-style FP8 checkpoint: e4m3 weight with one scale per 128 x 128 block."""
    from ipex_b200.utils.weight_only_quantization import _convert_woq_with_low_precision_checkpoint

    n, k, bn, bk = 320, 512, 128, 128  # N not a multiple of the block height
    rng = np.random.default_rng(31)
    w = torch.from_numpy((rng.standard_normal((n, k)) * 0.5).astype(np.float32)).to(torch.float8_e4m3fn)
    codes = w.view(torch.uint8).numpy()
    sinv = (rng.random(((n + bn - 1) // bn, k // bk)) * 0.02 + 0.01).astype(np.float32)
    sd = {"fc1.weight": w if store == "float8" else w.view(torch.uint8), "fc1.weight_scale_inv": torch.from_numpy(sinv),
          "lm_head.weight": torch.randn(32, n) * 0.05}
    model = TwoLinears(k, n, False)
    out = _convert_woq_with_low_precision_checkpoint(
        model, qmap(ipex), sd, {"quant_method": "fp8", "weight_block_size": [bn, bk]})
    assert out.fc1.dtype == ipex.quantization.WoqWeightDtype.FP8 and out.fc1._group_size == bk
    x = make_acts(6, k, seed=5)
    y = bf16_numpy(out.fc1(bf16_tensor(x, "cuda")))
    s_rows = np.repeat(sinv, bn, 0)[:n]
    ref = O.woq_linear_any(x, codes, s_rows, None, None, O.WOQ_DTYPE_FP8, bk, "bf16", "bf16")
    parity(y, ref)
    # The oracle's decoder against torch's own conversion of the same codes.  The reference's
    # decoder (csrc/cpu/aten/utils/woq.h:465-483) rebiases the exponent of every non-zero code,
    # so the 14 subnormal codes read as (1 + m/8) * 2^-7 instead of m/8 * 2^-6 and the two NaN
    # codes as +-480; oracle and kernel follow the reference there, on all other codes the three agree.
    normal = ((codes >> 3) & 15 != 0) & (codes & 127 != 127) | (codes & 127 == 0)
    assert normal.mean() > 0.9 and not normal.all()
    np.testing.assert_array_equal(O.fp8_e4m3_to_f32(codes)[normal], w.float().numpy()[normal])
    all_codes = np.arange(256, dtype=np.uint8)
    sub = ((all_codes >> 3) & 15 == 0) & (all_codes & 7 != 0)
    want = (1.0 + (all_codes[sub] & 7) / 8.0) * 2.0 ** -7 * np.where(all_codes[sub] & 128, -1.0, 1.0)
    np.testing.assert_array_equal(O.fp8_e4m3_to_f32(all_codes[sub]), want.astype(np.float32))


def test_checkpoint_and_config_must_agree(ipex):
    from ipex_b200.utils.weight_only_quantization import _convert_woq_with_low_precision_checkpoint

    with pytest.raises(AssertionError, match="do not match"):
        _convert_woq_with_low_precision_checkpoint(TwoLinears(64, 64, False), qmap(ipex),
                                                   {"fc1.weight": torch.zeros(64, 64)}, {"quant_method": "gptq"})
    with pytest.raises(AssertionError, match="not supported"):
        _convert_woq_with_low_precision_checkpoint(TwoLinears(64, 64, False), qmap(ipex), {}, {"quant_method": "rtn"})


def test_rmsnorm_quant_module_shares_one_quantisation(ipex):
    """_IPEXRmsNormQuantLinears(norm, [q, k, v]) == the three INT8-compute linears on
    rms_norm(x), each quantising for itself."""
    from ipex_b200.transformers.fusions.norm_quant import _IPEXRmsNormQuantLinears

    q = ipex.quantization
    qm = q.get_weight_only_quant_qconfig_mapping(weight_dtype=q.WoqWeightDtype.INT8, lowp_mode=q.WoqLowpMode.INT8,
                                                 act_quant_mode=q.WoqActQuantMode.PER_BATCH_SYM)
    mods = [woq(ipex, make_linear(n, 1024, False, 70 + i), qm) for i, n in enumerate((1024, 256, 256))]
    norm = nn.RMSNorm(1024, eps=1e-5)
    with torch.no_grad():
        norm.weight.copy_(torch.rand(1024) + 0.5)
    norm = norm.cuda().bfloat16()
    fused = _IPEXRmsNormQuantLinears(norm, mods)
    x = (torch.randn(3, 5, 1024, device="cuda") * 2).bfloat16()
    outs = fused(x)
    assert len(outs) == 3 and outs[0].shape == (3, 5, 1024) and outs[1].shape == (3, 5, 256)
    # reference: the library's own normalised rows, then every linear quantising for itself
    _, _, _, y = ipex._capi.rmsnorm_quant(x, norm.weight, 1e-5, 6, want_y=True)
    for got, mod in zip(outs, mods):
        assert torch.equal(got, mod(y.view(3, 5, 1024)))
    # and close to torch's own rms_norm feeding the same linears
    y_t = torch.nn.functional.rms_norm(x.float(), (1024,), norm.weight.float(), 1e-5).bfloat16()
    a, b = outs[0].float(), mods[0](y_t).float()
    assert (a - b).abs().max() <= 0.02 * b.abs().max()
