"""Llama-3-8B-architecture decode stack with INT4 group-128 weight-only-quantised linears
(`python bench.py --stack`).

32 layers, hidden 4096, 32 query heads / 8 KV heads of 128, SwiGLU FFN 14336, RMSNorm eps 1e-5,
RoPE theta 5e5, vocabulary 128256 with the language-model head kept in bf16; random weights
~N(0, 0.02), prompts of uniform-random token ids.  Every linear of the decoder layers is built
through ipex_b200.llm.optimize (quantise, prepack, fuse: q/k/v as one concatenated linear, gate
and up in one kernel with the silu*mul epilogue, the residual adds in the epilogues of o_proj and
down_proj).  Attention, RMSNorm, RoPE, the embedding, the head and the arg-max are stock
PyTorch: they are the harness, the linears are the thing measured.

For each batch size the prompt is prefilled into a static KV cache, then 128 greedy tokens are
decoded with one CUDA graph per decode step replayed once per token.  Reported per batch size:
prefill time, decode time per token, and the time the WOQ linears alone take per token (the same
modules at the same token count in a graph of their own), with that as weight bytes per second
against the measured HBM peak.
"""
import json
import math
import time

import torch
import torch.nn.functional as F
from torch import nn

HIDDEN, LAYERS, HEADS, KV_HEADS, HEAD_DIM, FFN, VOCAB = 4096, 32, 32, 8, 128, 14336, 128256
EPS, THETA, GROUP = 1e-5, 5e5, 128
PROMPT, NEW_TOKENS = 1024, 128


def woq_weight_bytes_per_layer():
    def wb(n, k):
        return n * k // 2 + 3 * n * (k // GROUP)

    return wb((HEADS + 2 * KV_HEADS) * HEAD_DIM, HIDDEN) + wb(HIDDEN, HIDDEN) + wb(2 * FFN, HIDDEN) + wb(HIDDEN, FFN)


class Attention(nn.Module):
    def __init__(self, dev):
        super().__init__()
        kw = dict(bias=False, device=dev, dtype=torch.bfloat16)
        self.q_proj = nn.Linear(HIDDEN, HEADS * HEAD_DIM, **kw)
        self.k_proj = nn.Linear(HIDDEN, KV_HEADS * HEAD_DIM, **kw)
        self.v_proj = nn.Linear(HIDDEN, KV_HEADS * HEAD_DIM, **kw)
        self.o_proj = nn.Linear(HEADS * HEAD_DIM, HIDDEN, **kw)


class Mlp(nn.Module):
    def __init__(self, dev):
        super().__init__()
        kw = dict(bias=False, device=dev, dtype=torch.bfloat16)
        self.gate_proj = nn.Linear(HIDDEN, FFN, **kw)
        self.up_proj = nn.Linear(HIDDEN, FFN, **kw)
        self.down_proj = nn.Linear(FFN, HIDDEN, **kw)
        self.act_fn = nn.SiLU()

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))


def rope(x, cos, sin):
    """x [B, heads, T, 128]; cos / sin [T, 64] (rotate-half convention)."""
    x1, x2 = x[..., :HEAD_DIM // 2], x[..., HEAD_DIM // 2:]
    c, s = cos[None, None], sin[None, None]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), -1)


class DecoderLayer(nn.Module):
    def __init__(self, dev):
        super().__init__()
        self.self_attn = Attention(dev)
        self.mlp = Mlp(dev)
        self.input_layernorm = nn.RMSNorm(HIDDEN, eps=EPS, device=dev, dtype=torch.bfloat16)
        self.post_attention_layernorm = nn.RMSNorm(HIDDEN, eps=EPS, device=dev, dtype=torch.bfloat16)

    def forward(self, x, cache_k, cache_v, pos, cos, sin, mask):
        """x [B, T, H].  pos: device int64 [T] (cache rows this call writes).  mask None = causal
        prefill from an empty cache, else bool [S_max] of the cache rows a decode token may see."""
        b, t, _ = x.shape
        a = self.self_attn
        h = self.input_layernorm(x)
        q = a.q_proj(h).view(b, t, HEADS, HEAD_DIM).transpose(1, 2)
        k = a.k_proj(h).view(b, t, KV_HEADS, HEAD_DIM).transpose(1, 2)
        v = a.v_proj(h).view(b, t, KV_HEADS, HEAD_DIM).transpose(1, 2)
        q, k = rope(q, cos, sin), rope(k, cos, sin)
        cache_k.index_copy_(2, pos, k)
        cache_v.index_copy_(2, pos, v)
        if mask is None:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        else:
            # one new token: the 4 query heads of a KV head attend to the same rows, so they
            # are passed as 4 "query positions" of that head and no key is expanded
            qg = q.reshape(b, KV_HEADS, HEADS // KV_HEADS, HEAD_DIM)
            o = F.scaled_dot_product_attention(qg, cache_k, cache_v, attn_mask=mask[None, None, None, :])
            o = o.reshape(b, HEADS, 1, HEAD_DIM)
        o = o.transpose(1, 2).reshape(b, t, HEADS * HEAD_DIM)
        if hasattr(self, "mha_linear_add"):
            x = self.mha_linear_add(o, x)
        else:
            x = x + a.o_proj(o)
        h = self.post_attention_layernorm(x)
        if hasattr(self, "mlp_linear_add"):
            return self.mlp_linear_add(self.mlp.gate_up_fused(h), x)
        return x + self.mlp(h)

    def woq_linears_only(self, h, o, act):
        """The four WOQ launches of this layer on stand-in inputs of the right shapes."""
        self.self_attn.qkv_concat.concat(h)
        self.mha_linear_add(o, h)
        self.mlp.gate_up_fused(h)
        self.mlp_linear_add(act, h)


def build_stack(ipex, dev, log):
    q = ipex.quantization
    qmap = q.get_weight_only_quant_qconfig_mapping(weight_dtype=q.WoqWeightDtype.INT4, lowp_mode=q.WoqLowpMode.BF16,
                                                   group_size=GROUP)
    gen = torch.Generator(device=dev).manual_seed(20240611)
    layers = []
    t0 = time.time()
    for i in range(LAYERS):
        layer = DecoderLayer(dev)
        for p in layer.parameters():
            if p.dim() == 2:
                p.data.normal_(0.0, 0.02, generator=gen)
        layers.append(ipex.llm.optimize(layer, dtype=torch.bfloat16, quantization_config=qmap, inplace=True, device=dev))
    log(f"stack: {LAYERS} layers quantised, prepacked and fused in {time.time() - t0:.1f} s")
    embed = torch.empty(VOCAB, HIDDEN, device=dev, dtype=torch.bfloat16).normal_(0.0, 0.02, generator=gen)
    head = torch.empty(VOCAB, HIDDEN, device=dev, dtype=torch.bfloat16).normal_(0.0, 0.02, generator=gen)
    norm = nn.RMSNorm(HIDDEN, eps=EPS, device=dev, dtype=torch.bfloat16)
    return layers, embed, head, norm


def check_layer(ipex, layer, dev):
    """Layer 0's fused WOQ linears against fp32 matmuls on the weights the contexts dequantise."""
    gen = torch.Generator(device=dev).manual_seed(5)
    worst = 0.0
    mods = [("qkv", layer.self_attn.qkv_concat.concat.concat_linear, None),
            ("o_proj", layer.self_attn.o_proj, None), ("down_proj", layer.mlp.down_proj, None)]
    for name, mod, _ in mods:
        ctx = mod._op_context
        n, k = ctx.get_weight_shape()
        x = torch.randn(8, k, device=dev, generator=gen).bfloat16()
        qw, z = ctx.get_weight(), ctx.get_zero_points().float().reshape(n, -1)
        s = ctx.get_scales().float().reshape(n, -1).bfloat16().float()  # the kernels multiply by the bf16 scale
        codes = torch.stack((qw & 15, qw >> 4), -1).reshape(n, k).float()
        w = ((codes - z.repeat_interleave(GROUP, 1)) * s.repeat_interleave(GROUP, 1)).bfloat16().float()
        ref = x.float() @ w.t()
        y = mod(x).float()
        err = ((y - ref).abs().max() / ref.abs().max()).item()
        worst = max(worst, err)
        if err > 1e-2:
            raise RuntimeError(f"stack check: {name} differs from the fp32 product of its dequantised weights by {err:.3e}")
    g = layer.mlp.gate_up_fused
    x = torch.randn(8, HIDDEN, device=dev, generator=gen).bfloat16()
    y = g(x)
    if y.shape != (8, FFN) or not torch.isfinite(y.float()).all():
        raise RuntimeError("stack check: fused gate/up output has the wrong shape or non-finite values")
    return worst


def run_stack(args, peaks, clock_sampler):
    """peaks() -> (HBM GB/s, bf16 TFLOP/s, "measured" | "fallback"); clock_sampler(gpu_index) samples
    nvidia-smi while the timed regions run.  Both come from bench.py."""
    import ipex_b200

    ipex_b200.load_ops()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)

    def log(msg):
        if args.verbose:
            print(msg, file=__import__("sys").stderr, flush=True)

    layers, embed, head, norm = build_stack(ipex_b200, dev, log)
    worst = check_layer(ipex_b200, layers[0], dev)
    log(f"stack: layer-0 linears agree with their dequantised weights (worst {worst:.2e} of the output range)")
    s_max = PROMPT + NEW_TOKENS
    inv = 1.0 / (THETA ** (torch.arange(0, HEAD_DIM, 2, device=dev, dtype=torch.float32) / HEAD_DIM))
    ang = torch.arange(s_max, device=dev, dtype=torch.float32)[:, None] * inv[None]
    cos_t, sin_t = ang.cos().bfloat16(), ang.sin().bfloat16()
    hbm_peak, _, peak_kind = peaks()
    wbytes = LAYERS * woq_weight_bytes_per_layer()
    batches = [int(b) for b in str(args.stack).split(",")] if args.stack not in (None, "all") else [1, 8, 32]
    new_tokens = args.new_tokens
    results = []
    sampler = clock_sampler(0)
    for bs in batches:
        gen = torch.Generator(device=dev).manual_seed(100 + bs)
        prompt = torch.randint(0, VOCAB, (bs, PROMPT), device=dev, generator=gen)
        cache_k = [torch.zeros(bs, KV_HEADS, s_max, HEAD_DIM, device=dev, dtype=torch.bfloat16) for _ in layers]
        cache_v = [torch.zeros_like(c) for c in cache_k]

        # ---- prefill, four sequences at a time -------------------------------------------
        tok = torch.empty(bs, dtype=torch.long, device=dev)
        ppos = torch.arange(PROMPT, device=dev)

        def prefill():
            for b0 in range(0, bs, 4):
                b1 = min(bs, b0 + 4)
                x = embed[prompt[b0:b1]]
                for i, layer in enumerate(layers):
                    x = layer(x, cache_k[i][b0:b1], cache_v[i][b0:b1], ppos, cos_t[:PROMPT], sin_t[:PROMPT], None)
                tok[b0:b1] = (norm(x[:, -1]) @ head.t()).argmax(-1)

        with torch.no_grad():
            prefill()  # warm-up: packs the second tiling of every layer on first use
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            prefill()
            e1.record()
            torch.cuda.synchronize()
            # a kernel that gave up a bounded wait still ends; its status word says so
            torch.ops.torch_ipex.woq_check_status()
        prefill_ms = e0.elapsed_time(e1)
        first = tok.clone()

        # ---- one decode step as a CUDA graph ---------------------------------------------
        pos = torch.full((1,), PROMPT, dtype=torch.long, device=dev)
        rows = torch.arange(s_max, device=dev)
        out_tokens = torch.zeros(new_tokens, bs, dtype=torch.long, device=dev)
        step_no = torch.zeros(1, dtype=torch.long, device=dev)

        def decode_step():
            x = embed[tok][:, None, :]
            cos, sin = cos_t.index_select(0, pos), sin_t.index_select(0, pos)
            mask = rows <= pos
            for i, layer in enumerate(layers):
                x = layer(x, cache_k[i], cache_v[i], pos, cos, sin, mask)
            nxt = (norm(x[:, 0]) @ head.t()).argmax(-1)
            tok.copy_(nxt)
            out_tokens.index_copy_(0, step_no, nxt[None])
            pos.add_(1)
            step_no.add_(1)

        side = torch.cuda.Stream()  # warm-up and capture share it: the ops' scratch is kept per stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(3):
                decode_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(graph, stream=side):
            decode_step()
        # warm-up replays, then the timed 128 greedy steps from the state the prefill left
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        tok.copy_(first)
        pos.fill_(PROMPT)
        step_no.zero_()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(new_tokens):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        decode_ms = e0.elapsed_time(e1) / new_tokens
        torch.ops.torch_ipex.woq_check_status()
        distinct = int(out_tokens.unique().numel())

        # ---- the WOQ linears of one token step alone -------------------------------------
        h = torch.randn(bs, HIDDEN, device=dev, generator=gen).bfloat16()
        o = torch.randn(bs, HIDDEN, device=dev, generator=gen).bfloat16()
        act = torch.randn(bs, FFN, device=dev, generator=gen).bfloat16()

        def linears_only():
            for layer in layers:
                layer.woq_linears_only(h, o, act)

        side.wait_stream(torch.cuda.current_stream())
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(3):
                linears_only()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        lgraph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(lgraph, stream=side):
            linears_only()
        for _ in range(3):
            lgraph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(new_tokens):
            lgraph.replay()
        e1.record()
        torch.cuda.synchronize()
        lin_ms = e0.elapsed_time(e1) / new_tokens
        gbps = wbytes / (lin_ms * 1e-3) / 1e9
        results.append({
            "batch": bs, "prefill_ms": round(prefill_ms, 2),
            "prefill_tokens_per_s": round(bs * PROMPT / (prefill_ms * 1e-3), 1),
            "decode_ms_per_token": round(decode_ms, 4),
            "decode_tokens_per_s": round(bs / (decode_ms * 1e-3), 1),
            "woq_linear_ms_per_token": round(lin_ms, 4),
            "woq_linear_share_of_step": round(lin_ms / decode_ms, 3),
            "woq_weight_GBps": round(gbps, 1),
            "roofline_frac": round(gbps / hbm_peak, 4),
            "distinct_tokens_generated": distinct,
        })
        log(f"stack: batch {bs}: {results[-1]}")
        del graph, lgraph, cache_k, cache_v
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    print(json.dumps({
        "metric": "llama3_8b_int4_woq_decode_stack", "unit": "ms/token", "higher_is_better": False,
        "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "Llama-3-8B architecture, 32 layers, INT4 asymmetric group-128 WOQ on all decoder "
                               "linears (lm_head bf16), prompt %d, %d greedy steps, static KV cache, CUDA-graph "
                               "decode step" % (PROMPT, new_tokens),
                   "woq_launches_per_token": 4 * LAYERS, "woq_weight_bytes_per_token": wbytes,
                   "inputs": "larger than L2 (%.1f GB of packed weights read per token)" % (wbytes / 1e9)},
        "roofline_peak_GBps": hbm_peak, "roofline_peak_kind": peak_kind, "results": results, "checked": True,
        "check": {"layer0_linears_vs_dequantised_fp32_worst_rel_to_range": round(worst, 5)},
        "clocks": clocks,
    }))
    assert math.isfinite(results[0]["decode_ms_per_token"])
