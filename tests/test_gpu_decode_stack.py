"""A Llama-architecture decode stack in miniature (RMSNorm, RoPE, grouped-query attention, SwiGLU,
bf16 lm_head) whose linears are INT4 group-128 weight-only quantised through
ipex_b200.llm.optimize and the reference's fusion modules, against the same stack with the
oracle's dequantised bf16 weights in stock torch linears.  Prompt pass (prefill-size M) followed
by greedy decode steps with a KV cache (decode-size M): the architecture of the Llama-3-8B
configuration at a size a unit test can afford; attention, norm and RoPE are stock torch."""
import copy

import pytest
import torch
import torch.nn.functional as F
from torch import nn

from oracle import woq_oracle as O

pytestmark = pytest.mark.gpu

HID, NQ, NKV, HD, FFN, LAYERS, VOCAB, GROUP = 512, 4, 2, 128, 1536, 3, 1024, 128


@pytest.fixture(scope="module")
def ipex():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ipex_b200

    ipex_b200.load_ops()
    return ipex_b200


class RMSNorm(nn.Module):
    def __init__(self, n, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(n))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope(x, pos, theta=5e5):
    # x [B, H, T, D], pos [T]
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x.float()[..., ::2], x.float()[..., 1::2]
    out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)
    return out.to(x.dtype)


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.ln1, self.ln2 = RMSNorm(HID), RMSNorm(HID)
        self.qkv = nn.Linear(HID, (NQ + 2 * NKV) * HD, bias=False)
        self.o_proj = nn.Linear(NQ * HD, HID, bias=False)
        self.gate = nn.Linear(HID, FFN, bias=False)
        self.up = nn.Linear(HID, FFN, bias=False)
        self.down = nn.Linear(FFN, HID, bias=False)

    def mlp(self, h):
        return self.down(F.silu(self.gate(h)) * self.up(h))

    def forward(self, x, pos, cache):
        b, t, _ = x.shape
        qkv = self.qkv(self.ln1(x)).view(b, t, NQ + 2 * NKV, HD).transpose(1, 2)
        q, k, v = qkv[:, :NQ], qkv[:, NQ:NQ + NKV], qkv[:, NQ + NKV:]
        q, k = rope(q, pos), rope(k, pos)
        if cache is not None:
            k = torch.cat([cache[0], k], dim=2)
            v = torch.cat([cache[1], v], dim=2)
        rep = NQ // NKV
        att = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1),
                                             is_causal=cache is None)
        x = x + self.o_proj(att.transpose(1, 2).reshape(b, t, NQ * HD))
        x = x + self.mlp(self.ln2(x))
        return x, (k, v)


class Stack(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(VOCAB, HID)
        self.layers = nn.ModuleList(Block() for _ in range(LAYERS))
        self.norm = RMSNorm(HID)
        self.lm_head = nn.Linear(HID, VOCAB, bias=False)

    def forward(self, ids, pos, caches):
        x = self.embed(ids)
        new = []
        for i, layer in enumerate(self.layers):
            x, c = layer(x, pos, None if caches is None else caches[i])
            new.append(c)
        return self.lm_head(self.norm(x)), new


class FusedMlpBlock(Block):
    """The block with the reference's fusion modules around the WOQ linears: silu(gate)*up as
    woq_linear_silu + woq_linear_mul, the residual adds fused into o_proj and down."""

    def adopt(self, ipex):
        from ipex_b200.transformers.fusions import linear_fusion as fus

        self.mlp_silu_mul = fus._IPEXlinearSiluMul(self.gate, self.up)
        self.o_add = fus._IPEXlinearAdd(self.o_proj)
        self.down_add = fus._IPEXlinearAdd(self.down)
        return self

    def forward(self, x, pos, cache):
        b, t, _ = x.shape
        qkv = self.qkv(self.ln1(x)).view(b, t, NQ + 2 * NKV, HD).transpose(1, 2)
        q, k, v = qkv[:, :NQ], qkv[:, NQ:NQ + NKV], qkv[:, NQ + NKV:]
        q, k = rope(q, pos), rope(k, pos)
        if cache is not None:
            k = torch.cat([cache[0], k], dim=2)
            v = torch.cat([cache[1], v], dim=2)
        rep = NQ // NKV
        att = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1),
                                             is_causal=cache is None)
        x = self.o_add(att.transpose(1, 2).reshape(b, t, NQ * HD), x)
        x = self.down_add(self.mlp_silu_mul(self.ln2(x)), x)
        return x, (k, v)


def dequantised_copy(model, ipex):
    """Same stack, every block linear replaced by an nn.Linear holding the oracle's
    bf16((q - zp) * bf16(scale)) weights of the codes the package's quantiser produces."""
    q = ipex.quantization
    ref = copy.deepcopy(model)
    for blk in ref.layers:
        for name in ("qkv", "o_proj", "gate", "up", "down"):
            lin = getattr(blk, name)
            qw, s, z = q.quantize_per_block(lin.weight.detach().float().cuda(), q.WoqWeightDtype.INT4, GROUP)
            w = O.dequantize_weight(qw.cpu().numpy(), s.half().cpu().numpy(), z.cpu().numpy(), O.WOQ_DTYPE_INT4,
                                    lin.in_features, GROUP)
            lin.weight.data = torch.from_numpy(w)
    return ref.cuda().bfloat16().eval()


@pytest.mark.parametrize("batch", [1, 8])
def test_prompt_then_greedy_decode(ipex, batch):
    torch.manual_seed(1234)
    model = Stack().eval()
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() == 2:
                p.normal_(0, 0.02)
    ref = dequantised_copy(model, ipex)

    q = ipex.quantization
    qmap = q.get_weight_only_quant_qconfig_mapping(weight_dtype=q.WoqWeightDtype.INT4,
                                                   lowp_mode=q.WoqLowpMode.BF16, group_size=GROUP)
    fused = copy.deepcopy(model)
    for i, blk in enumerate(fused.layers):
        blk.__class__ = FusedMlpBlock
    woq = ipex.llm.optimize(fused, dtype=torch.bfloat16, quantization_config=qmap, inplace=True)
    W = ipex.nn.modules.WeightOnlyQuantizedLinear
    for blk in woq.layers:
        assert all(isinstance(getattr(blk, n), W) for n in ("qkv", "o_proj", "gate", "up", "down"))
        blk.adopt(ipex)
    assert isinstance(woq.lm_head, nn.Linear)  # kept in bf16

    prompt_len, steps = 40, 6
    ids = torch.randint(0, VOCAB, (batch, prompt_len), device="cuda")
    same_tokens = 0
    with torch.no_grad():
        pos = torch.arange(prompt_len, device="cuda")
        lg_w, cache_w = woq(ids, pos, None)       # M = batch * 40 tokens: prefill-size linears
        lg_r, cache_r = ref(ids, pos, None)
        for step in range(steps):
            a, b = lg_w[:, -1].float(), lg_r[:, -1].float()
            # the two stacks differ by summation order inside the linears only
            rel = (a - b).abs().mean() / b.abs().mean()
            assert rel < 2e-2, (step, float(rel))
            assert F.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.999
            tok_w, tok_r = a.argmax(-1), b.argmax(-1)
            same_tokens += int((tok_w == tok_r).sum())
            nxt = tok_r[:, None]                  # both continue from the reference's token
            pos = torch.tensor([prompt_len + step], device="cuda")
            lg_w, cache_w = woq(nxt, pos, cache_w)  # M = batch tokens: decode-size linears
            lg_r, cache_r = ref(nxt, pos, cache_r)
    assert same_tokens >= int(0.7 * batch * steps), same_tokens  # random-init logits are nearly flat
