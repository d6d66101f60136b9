"""Mixtral-style mixture-of-experts layer built from WOQ linears (config: 8 experts, top-2 softmax
router, SwiGLU experts, INT4 group-128), checked against the oracle's restatement of the reference
loop (csrc/cpu/aten/kernels/MoEKrnl.cpp:67-285; reference/modules/decoder.py:919-962)."""
import numpy as np
import pytest
import torch

from oracle import woq_oracle as O
from tests.helpers import bf16_numpy, bf16_tensor, make_acts

pytestmark = pytest.mark.gpu

E, G = 8, 128


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ipex_b200

    ipex_b200.load_ops()
    return ipex_b200


def make_experts(hidden, ffn, seed):
    rng = np.random.default_rng(seed)
    experts = []
    for e in range(E):
        w13 = (rng.standard_normal((2 * ffn, hidden)) * 0.02).astype(np.float32)
        w2 = (rng.standard_normal((hidden, ffn)) * 0.02).astype(np.float32)
        q13 = O.quantize_per_block(w13, O.WOQ_DTYPE_INT4, G)
        q2 = O.quantize_per_block(w2, O.WOQ_DTYPE_INT4, G)
        experts.append({"w13": (q13[0], q13[1].astype(np.float16), q13[2]),
                        "w2": (q2[0], q2[1].astype(np.float16), q2[2])})
    router = (rng.standard_normal((E, hidden)) * 0.02).astype(np.float32)
    return experts, O.rne_bf16(router)


def parity(y, y_ref):
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx <= O.MAX_ABS_TOL and mr <= O.MEAN_REL_TOL, (mx, mr)  # measured: at most 3e-6


@pytest.mark.parametrize("tokens", [1, 16, 256])
def test_moe_layer_c_abi(env, tokens):
    capi = env._capi
    hidden, ffn = 512, 1024
    experts, router = make_experts(hidden, ffn, seed=4000)
    h = make_acts(tokens, hidden, seed=4000 + tokens)
    idx, w = O.moe_route_top2(h, router)
    ref = O.moe_layer(h, idx, w, experts, G)
    hg = bf16_tensor(h, "cuda")
    out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    ctxs = []
    for ex in experts:
        q, s, z = ex["w13"]
        c13 = capi.WoqContext(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(),
                              None, 2 * ffn, hidden, capi.DTYPE_INT4, G, capi.LOWP_BF16,
                              layout_flags=capi.LAYOUT_GATE_UP)
        q, s, z = ex["w2"]
        c2 = capi.WoqContext(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(),
                             None, hidden, ffn, capi.DTYPE_INT4, G, capi.LOWP_BF16)
        ctxs.append((c13, c2))
    ws = None
    for e, (c13, c2) in enumerate(ctxs):
        t_sel, j_sel = np.nonzero(idx == e)
        if t_sel.size == 0:
            continue
        ti = torch.from_numpy(t_sel.astype(np.int32)).cuda()
        tw = bf16_tensor(w[t_sel, j_sel], "cuda")
        ws = capi.moe_expert(c13, c2, hg, ti, tw, out, ws)
    ws.status()
    parity(bf16_numpy(out), ref)


@pytest.mark.parametrize("tokens", [4, 64])
def test_mixtral_moe_woq_operator(env, tokens):
    """The reference's per-expert operator with separate w1 / w3 / w2 contexts."""
    hidden, ffn = 512, 1024
    experts, router = make_experts(hidden, ffn, seed=4100)
    h = make_acts(tokens, hidden, seed=4100 + tokens)
    idx, w = O.moe_route_top2(h, router)
    ref = O.moe_layer(h, idx, w, experts, G)
    hg = bf16_tensor(h, "cuda")
    out = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    rw = bf16_tensor(w, "cuda")
    sel = torch.from_numpy(idx.astype(np.int64)).cuda()
    expert_mask = torch.nn.functional.one_hot(sel, num_classes=E).permute(2, 1, 0)

    def ctx(q, s, z, n, k):
        return torch.ops.ipex_prepack.weight_only_qlinear_prepack(
            torch.from_numpy(q).cuda(), 2, [n, k], torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(),
            None, None, None, G, 2, -1)

    keep = []
    for e, ex in enumerate(experts):
        q, s, z = ex["w13"]
        c1, c3 = ctx(q[:ffn], s[:ffn], z[:ffn], ffn, hidden), ctx(q[ffn:], s[ffn:], z[ffn:], ffn, hidden)
        q, s, z = ex["w2"]
        c2 = ctx(q, s, z, hidden, ffn)
        keep += [c1, c2, c3]
        j, top_x = torch.where(expert_mask[e])
        out = torch.ops.torch_ipex.mixtral_moe_woq(hg, top_x, j, c1.get_data_handle(), c3.get_data_handle(),
                                                   c2.get_data_handle(), rw, out, False)
    parity(bf16_numpy(out), ref)


@pytest.mark.parametrize("tokens", [3, 40])
def test_deepseek_moe_woq_operator(env, tokens):
    """The list-of-contexts form (csrc/cpu/aten/MoE.cpp:290-330): same result as the per-expert operator
    called expert by expert, experts nobody chose are skipped."""
    hidden, ffn = 512, 1024
    experts, router = make_experts(hidden, ffn, seed=4200)
    h = make_acts(tokens, hidden, seed=4200 + tokens)
    idx, w = O.moe_route_top2(h, router)
    ref = O.moe_layer(h, idx, w, experts, G)
    hg = bf16_tensor(h, "cuda")
    rw = bf16_tensor(w, "cuda")
    sel = torch.from_numpy(idx.astype(np.int64)).cuda()

    def ctx(q, s, z, n, k):
        return torch.ops.ipex_prepack.weight_only_qlinear_prepack(
            torch.from_numpy(q).cuda(), 2, [n, k], torch.from_numpy(s).cuda(), torch.from_numpy(z).cuda(),
            None, None, None, G, 2, -1)

    gate, up, down = [], [], []
    for ex in experts:
        q, s, z = ex["w13"]
        gate.append(ctx(q[:ffn], s[:ffn], z[:ffn], ffn, hidden))
        up.append(ctx(q[ffn:], s[ffn:], z[ffn:], ffn, hidden))
        q, s, z = ex["w2"]
        down.append(ctx(q, s, z, hidden, ffn))
    out = torch.ops.torch_ipex.deepseek_moe_woq(hg, sel, gate, up, down, rw, False)
    parity(bf16_numpy(out), ref)
    # expert by expert through the per-expert operator: the same launches in the same order
    out2 = torch.zeros_like(out)
    expert_mask = torch.nn.functional.one_hot(sel, num_classes=E).permute(2, 1, 0)
    for e in range(E):
        j, top_x = torch.where(expert_mask[e])
        out2 = torch.ops.torch_ipex.mixtral_moe_woq(hg, top_x, j, gate[e].get_data_handle(), up[e].get_data_handle(),
                                                    down[e].get_data_handle(), rw, out2, False)
    assert (out.float() - out2.float()).abs().max() <= 2.0 ** -7 * out2.float().abs().max()


def test_config4_expert_shapes_one_token(env):
    """Full Mixtral-8x7B expert shapes (w13 28672x4096, w2 4096x14336), one token, two experts."""
    capi = env._capi
    hidden, ffn = 4096, 14336
    rng = np.random.default_rng(7)
    h = make_acts(1, hidden, seed=1)
    hg = bf16_tensor(h, "cuda")
    out = torch.zeros((1, hidden), dtype=torch.bfloat16, device="cuda")
    acc = np.zeros((1, hidden), dtype=np.float32)
    for e, wt in enumerate((0.625, 0.375)):
        g = torch.Generator(device="cuda").manual_seed(e)
        w13 = torch.randn((2 * ffn, hidden), device="cuda", generator=g) * 0.02
        w2 = torch.randn((hidden, ffn), device="cuda", generator=g) * 0.02
        q13 = env.quantization.quantize_per_block(w13, 2, G)
        q2 = env.quantization.quantize_per_block(w2, 2, G)
        c13 = capi.WoqContext(q13[0], q13[1].half(), q13[2], None, 2 * ffn, hidden, capi.DTYPE_INT4, G,
                              capi.LOWP_BF16, layout_flags=capi.LAYOUT_GATE_UP)
        c2 = capi.WoqContext(q2[0], q2[1].half(), q2[2], None, hidden, ffn, capi.DTYPE_INT4, G, capi.LOWP_BF16)
        ti = torch.zeros(1, dtype=torch.int32, device="cuda")
        tw = torch.tensor([wt], device="cuda").bfloat16()
        capi.moe_expert(c13, c2, hg, ti, tw, out).status()
        a = O.woq_linear_bf16(h, q13[0].cpu().numpy(), q13[1].half().cpu().numpy(), q13[2].cpu().numpy(), None,
                              O.WOQ_DTYPE_INT4, G, O.FUSE_SILU_MUL)
        y = O.woq_linear_bf16(a, q2[0].cpu().numpy(), q2[1].half().cpu().numpy(), q2[2].cpu().numpy(), None,
                              O.WOQ_DTYPE_INT4, G)
        acc = O.rne_bf16(acc + y * np.float32(wt))
    parity(bf16_numpy(out), acc)
