#!/usr/bin/env python
"""Benchmark of the INT4 weight-only-quantised linear hot path.

Workload (synthetic, seeded): the linears of a Llama-3-70B-architecture decoder, INT4
asymmetric group-128, 80 layers x {QKV 10240x8192, o_proj 8192x8192, gate_up 57344x8192 with
the silu*mul epilogue, down_proj 8192x28672}, decode batch M tokens (default 1).  A step is one
token step through all 320 linears.  With N GPUs the layers are tensor-parallel: QKV / gate_up
sharded along N with an all-gather, o_proj / down_proj sharded along K with an all-reduce (NCCL).

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nproc-per-node 8 ... bench.py --gpus 8 --steps 20 --warmup 3
    python bench.py --impl reference          # the CPU restatement of the reference kernel

Prints ONE JSON line (rank 0).  `value` = weight bytes streamed per second over all GPUs
(inputs resident in HBM); `e2e` = the same through the public module API with the step's
activations copied from pinned host memory and the result copied back every step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG_DIR = os.path.join(ROOT, "intel-extension-for-pytorch_b200")
for _p in (ROOT, PKG_DIR):
    if _p not in sys.path:
        sys.path.insert(0, _p)

HIDDEN, QKV_N, FFN, LAYERS, GROUP = 8192, 10240, 28672, 80, 128
METRIC = "int4_woq_linear_weight_GBps_decode"
# DRAM bytes (read + write) per algorithmic byte of the decode kernel, from an ncu capture of a
# gate_up-sized launch (the device keeps 4 bytes of scale and zero point per row and group
# against 3 algorithmic ones, and split-K partial tiles are written and read back); the
# traffic of a launch grows in proportion to its bytes.
TRAFFIC_RATIO = 1.034
FUSED_MAX_TOKENS = 8  # --collective auto: largest decode batch that takes the fused exchange
UNIT = "GB/s"


def weight_bytes(n, k, g=GROUP):
    """Algorithmic weight bytes of one INT4 linear: nibbles + fp16 scale + u8 zero point."""
    return n * k // 2 + 3 * n * (k // g)


def layer_shapes(p):
    """(name, N_local, K_local, parallel kind) for one rank of a p-way tensor-parallel layer."""
    return [
        ("qkv", QKV_N // p, HIDDEN, "col"),
        ("o_proj", HIDDEN, HIDDEN // p, "row"),
        ("gate_up", 2 * FFN // p, HIDDEN, "col"),
        ("down_proj", HIDDEN, FFN // p, "row"),
    ]


def full_layer_weight_bytes():
    return sum(weight_bytes(n, k) for _, n, k, _ in layer_shapes(1))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6),
                              ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the reference's WOQ kernel on the host cores
# ------------------------------------------------------------------------------------------
def host_cpu():
    """Model name, logical CPUs and the ISA flags that matter for the reference's WOQ kernels."""
    model, flags = "unknown", []
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name") and model == "unknown":
                model = line.split(":", 1)[1].strip()
            elif line.startswith("flags") and not flags:
                have = set(line.split(":", 1)[1].split())
                flags = [f for f in ("avx2", "avx512f", "avx512bw", "avx512_vnni", "avx512_bf16", "avx512_fp16",
                                     "amx_bf16", "amx_int8") if f in have]
    except OSError:
        pass
    return {"model": model, "logical_cpus": os.cpu_count(), "isa": flags}


def cpu_baseline(m, warmup=5, passes=20):
    """Times the C restatement of the reference's CPU kernel (oracle/woq_oracle_c.c, OpenMP on
    every logical CPU of the host, set explicitly: a launcher's OMP_NUM_THREADS does not apply)
    on one of the 80 layers.  Fewer than 5 tokens take the reference's fp16 small-M microkernel
    (AVX512-FP16 intrinsics) where the CPU has it, as the reference's own dispatch does; otherwise
    the bf16 tile kernel.  Median of `passes` passes after `warmup` warm-up passes."""
    import numpy as np

    from oracle import woq_oracle_c as OC

    threads = os.cpu_count() or 1
    small = m < 5 and OC.has_fp16_kernel()
    rng = np.random.default_rng(0)
    layers = []
    for name, n, k, _ in layer_shapes(1):
        qw = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
        s = (rng.random((n, k // GROUP), dtype=np.float32) * 0.01 + 0.001).astype(np.float16).astype(np.float32)
        z = rng.integers(0, 16, (n, k // GROUP)).astype(np.float32)
        layers.append((name, OC.Layer(qw, n, k, s, z, None, GROUP), n, k))
    xs = {k: (rng.standard_normal((m, k)).astype(np.float32)) for k in (HIDDEN, FFN)}

    def one_pass():
        for _, L, n, k in layers:
            fusion = 0x100 if n == 2 * FFN else 0
            if small:
                L.linear_fp16_small_m(xs[k], fusion, threads=threads)
            else:
                L.linear_bf16(xs[k], fusion, threads=threads)

    for _ in range(max(1, warmup)):
        one_pass()
    times = []
    for _ in range(max(1, passes)):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    gbps = full_layer_weight_bytes() / dt / 1e9
    kernel = ("fp16 small-M microkernel, AVX512-FP16 intrinsics (the reference's route for M < 5)" if small
              else "bf16 tile-dequant + block GEMM, compiler-vectorised loops")
    return {"value": gbps, "unit": UNIT, "cores": threads, "kind": "port", "cpu": host_cpu(), "kernel": kernel,
            "sample": f"1 of {LAYERS} layers (4 linears, {full_layer_weight_bytes() / 1e6:.0f} MB of "
                      f"weights), M={m}, median of {passes} passes after {warmup} warm-up, blocked-layout C "
                      f"restatement of the reference kernel with OpenMP on {threads} threads"}, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    cb, dt = cpu_baseline(args.m, warmup=max(5, warm), passes=max(20, steps))
    line = {
        "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt * 1e3 * LAYERS, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {"workload": "llama3-70b linears, INT4 asym g128, decode", "m": args.m,
                   "layers": LAYERS, "note": "each step = a bounded sample (1 layer) of the workload; "
                   "ms_per_step extrapolates to 80 layers"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def build_layers(torch, capi, quant, p, rank, n_layers, device, m=1):
    """Random-init N(0, 0.02) weights, quantised on the GPU, packed into contexts."""
    layers = []
    for l in range(n_layers):
        row = {}
        for name, n, k, kind in layer_shapes(p):
            g = torch.Generator(device=device).manual_seed(1000 * l + 17 * rank + len(row))
            w = torch.randn((n, k), device=device, generator=g) * 0.02
            qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
            del w
            # one tiling is enough: the streaming one for decode sizes, the tensor-core one above
            flags = (capi.LAYOUT_STREAM_ONLY if m <= 16 else capi.LAYOUT_TC_ONLY) | capi.LAYOUT_DEFER_CHECK | (
                capi.LAYOUT_GATE_UP if name == "gate_up" else 0)
            row[name] = capi.WoqContext(qw, s.half(), z, None, n, k, capi.DTYPE_INT4, GROUP,
                                        capi.LOWP_BF16, layout_flags=flags)
            del qw, s, z
        layers.append(row)
    torch.cuda.synchronize()
    return layers


def _parity(torch, y, ref):
    """max |y - ref| / ||ref||_inf and mean |y - ref| / mean |ref| (the tolerances of the tests:
    1e-2 and 2e-3)."""
    y, ref = y.float(), ref.float()
    d = (y - ref).abs()
    return float(d.max() / ref.abs().max()), float(d.mean() / ref.abs().mean())


def _elementwise_rel(torch, y, ref):
    """Mean of |y - ref| / |ref| over the elements with |ref| > 1e-2 * ||ref||_inf: the stricter
    reading of "mean relative error", reported beside the ratio of means."""
    y, ref = y.float(), ref.float()
    keep = ref.abs() > 1e-2 * ref.abs().max()
    return float(((y - ref).abs()[keep] / ref.abs()[keep]).mean()) if bool(keep.any()) else 0.0


def verify_step(torch, dist, capi, L, p, rank, m, ws, hidden, resid, attn_slice, fused, comm, act_off,
                qkv_out, o_out, act_out, d_out):
    """Checks what the eager step left behind for the LAST layer (every layer gets the same
    inputs, so the output buffers hold the last layer's results) before anything is timed.
    The yardstick is a plain fp32 matmul on the layer's dequantised weights (dumped by the
    library, which the tests pin bit for bit to the CPU oracle), with the partial sums of a
    row-parallel layer added across ranks in fp32.  With N > 1 it also checks that every rank
    holds the same bits.  Raises on a mismatch; returns the figures for the JSON line."""
    bf = torch.bfloat16

    def deq(ctx):
        return ctx.dump_dequant().float()

    def silu_mul(y):
        half = y.shape[-1] // 2
        gate, up = y[:, :half].to(bf).float(), y[:, half:].to(bf).float()
        sig = torch.sigmoid(gate).to(bf).float()
        return ((gate * sig).to(bf).float() * up).to(bf)

    def reduce_ranks(t):
        if p > 1:
            dist.all_reduce(t)
        return t

    def gather_ranks(t):
        if p == 1:
            return t
        out = torch.empty((p,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous())
        return out.permute(1, 0, 2).reshape(t.shape[0], -1)

    if fused:
        qkv_out = comm.gathered(0, m, QKV_N)
        act_out = comm.gathered(act_off, m, FFN)
    else:
        # NCCL path: [p, m, n/p] buffers (or the local [m, n] ones on one GPU)
        if p > 1:
            qkv_out = qkv_out.permute(1, 0, 2).reshape(m, -1)
            act_out = act_out.permute(1, 0, 2).reshape(m, -1)
    worst = [0.0, 0.0, 0.0]

    def compare(name, y, ref):
        mx, mr = _parity(torch, y, ref)
        worst[0], worst[1] = max(worst[0], mx), max(worst[1], mr)
        worst[2] = max(worst[2], _elementwise_rel(torch, y, ref))
        # The comparison arm sums the ranks' bf16 partials with NCCL in bf16, rounding after every
        # addition (2.5e-3 mean relative at 8 ranks); the fused exchange adds them in fp32 and
        # rounds once, like the yardstick.  The NCCL arm's row-parallel outputs get twice the bar.
        bar = 4e-3 if (p > 1 and not fused and name in ("o_proj", "down_proj")) else 2e-3
        if not (mx <= 1e-2 and mr <= bar):
            raise RuntimeError(f"bench check failed on rank {rank}: {name} max-abs/inf {mx:.3e}, mean-rel {mr:.3e}")

    qkv_ref = gather_ranks((hidden.float() @ deq(L["qkv"]).T).to(bf))
    compare("qkv", qkv_out, qkv_ref)
    o_part = (attn_slice.float() @ deq(L["o_proj"]).T)
    o_ref = (reduce_ranks(o_part.to(bf).float() if p > 1 else o_part).to(bf).float() + resid.float()).to(bf)
    compare("o_proj", o_out, o_ref)
    act_ref = gather_ranks(silu_mul(o_out.float() @ deq(L["gate_up"]).T))
    compare("gate_up", act_out, act_ref)
    act_mine = act_out[:, rank * (FFN // p):(rank + 1) * (FFN // p)]
    d_part = (act_mine.float() @ deq(L["down_proj"]).T)
    d_ref = (reduce_ranks(d_part.to(bf).float() if p > 1 else d_part).to(bf).float() + resid.float()).to(bf)
    compare("down_proj", d_out, d_ref)
    identical = True
    if p > 1:
        sums = torch.stack([t.contiguous().view(torch.int16).to(torch.int64).sum()
                            for t in (qkv_out, o_out, act_out, d_out)])
        every = torch.empty((p, 4), dtype=torch.int64, device=sums.device)
        dist.all_gather_into_tensor(every, sums)
        identical = bool((every == every[0]).all())
        if not identical:
            raise RuntimeError(f"bench check failed: ranks hold different output bits: {every.tolist()}")
    ws.status()
    torch.cuda.empty_cache()
    return {"max_abs_over_inf": worst[0], "mean_rel": worst[1], "mean_rel_elementwise": worst[2],
            "ranks_identical": identical,
            "against": "fp32 matmul on the dequantised weights of the last layer, partial sums added over ranks in fp32"}


def e2e_through_ops(torch, quant, m, device, n_layers=4, steps=20):
    """The step of `n_layers` layers through the registered operators (torch.ops.torch_ipex.*
    on contexts made by torch.ops.ipex_prepack.*), host activations in and host result out every
    step, eager (no CUDA graph): what a caller of the reference's op surface pays per call."""
    from ipex_b200 import _ops

    _ops.load_ops()
    pre = torch.ops.ipex_prepack
    ops = torch.ops.torch_ipex
    layers = []
    for l in range(n_layers):
        row = {}
        for name, n, k, _ in layer_shapes(1):
            g = torch.Generator(device=device).manual_seed(5000 + 10 * l + len(row))
            w = torch.randn((n, k), device=device, generator=g) * 0.02
            qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
            del w
            if name == "gate_up":
                row[name] = pre.weight_only_qlinear_prepack_gate_up(qw, 2, [n, k], s.half(), z, None, GROUP, 2, -1)
            else:
                row[name] = pre.weight_only_qlinear_prepack(qw, 2, [n, k], s.half(), z, None, None, None, GROUP, 2,
                                                            -1, False)
            del qw, s, z
        layers.append({k_: (v, v.get_data_handle()) for k_, v in row.items()})
    bf = dict(dtype=torch.bfloat16, device=device)
    hidden = torch.empty((m, HIDDEN), **bf)
    resid = torch.randn((m, HIDDEN), **bf)
    attn = torch.randn((m, HIDDEN), **bf)
    x_host = torch.randn((m, HIDDEN)).bfloat16().pin_memory()
    y_host = torch.empty((m, HIDDEN), dtype=torch.bfloat16).pin_memory()

    def step():
        hidden.copy_(x_host, non_blocking=True)
        d = None
        for L in layers:
            ops.ipex_woq_linear(hidden, L["qkv"][1])
            o = ops.woq_linear_add(attn, L["o_proj"][1], [resid])
            a = ops.woq_linear_silu_mul(o, L["gate_up"][1])
            d = ops.woq_linear_add(a, L["down_proj"][1], [resid])
        y_host.copy_(d, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    ops.woq_check_status()
    del layers
    torch.cuda.empty_cache()
    return {"value": full_layer_weight_bytes() * n_layers / dt / 1e9, "unit": UNIT, "layers": n_layers,
            "ms_per_step": dt * 1e3, "us_per_linear": dt * 1e6 / (4 * n_layers), "cuda_graph": False,
            "h2d_bytes_per_step": m * HIDDEN * 2, "d2h_bytes_per_step": m * HIDDEN * 2,
            "api": "torch.ops.torch_ipex.{ipex_woq_linear, woq_linear_add, woq_linear_silu_mul}"}


def fast_side_line(torch, capi, quant, device, m):
    """One Llama-3-70B layer's four linears with both INT4 dequantisers of the streaming kernel:
    the default (bf16 rounding per weight, the reference's tile dequantiser) and the hint
    WOQ_B200_HINT_STREAM_FAST (scale and zero point applied after each k-block sum).  Timed as a
    CUDA graph of the four launches in layer order (428 MB of weights per pass, more than L2);
    the deviation is mean |y_fast - y_default| / mean |y_default| per shape."""
    bf = dict(device=device, dtype=torch.bfloat16)
    hbm_peak, _, _ = peaks()
    sets = {}
    xs, ys = {}, {}
    g = torch.Generator(device=device).manual_seed(777)
    for name, n, k, _ in layer_shapes(1):
        w = torch.randn((n, k), device=device, generator=g) * 0.02
        qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
        del w
        flags = capi.LAYOUT_STREAM_ONLY | (capi.LAYOUT_GATE_UP if name == "gate_up" else 0)
        for hint in (capi.HINT_AUTO, capi.HINT_STREAM_FAST):
            sets.setdefault(hint, {})[name] = capi.WoqContext(qw, s.half(), z, None, n, k, capi.DTYPE_INT4, GROUP,
                                                              capi.LOWP_BF16, layout_flags=flags, kernel_hint=hint)
        xs[name] = torch.randn((m, k), generator=g, **bf)
        ys[name] = torch.empty((m, n // 2 if name == "gate_up" else n), **bf)
        del qw, s, z
    ws = capi.Workspace(max(c.workspace_bytes(m) for c in sets[capi.HINT_AUTO].values()), device)
    out = {"m": m, "shapes": {}}
    results = {}
    for hint, key in ((capi.HINT_AUTO, "per_weight"), (capi.HINT_STREAM_FAST, "after_sum")):
        def layer():
            for name in ("qkv", "o_proj", "gate_up", "down_proj"):
                sets[hint][name].linear(xs[name], capi.FUSE_SILU_MUL if name == "gate_up" else capi.FUSE_NONE,
                                        out=ys[name], workspace=ws)
        layer()
        torch.cuda.synchronize()
        results[key] = {name: ys[name].float().clone() for name in ys}
        us = _time_graph(torch, layer, 4) * 4
        wb = full_layer_weight_bytes()
        out[key] = {"layer_us": round(us, 2), "weight_GBps": round(wb / us / 1e3, 1),
                    "frac": round(wb / us / 1e3 / hbm_peak, 4)}
    ws.status()
    for name in ys:
        a, b = results["after_sum"][name], results["per_weight"][name]
        out["shapes"][name] = {"mean_rel_deviation": float((a - b).abs().mean() / b.abs().mean()),
                               "max_abs_over_inf_norm": float((a - b).abs().max() / b.abs().max())}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from ipex_b200 import _capi as capi
    from ipex_b200 import quantization as quant

    p = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert p == args.gpus or p == 1, f"--gpus {args.gpus} but WORLD_SIZE={p}"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    def log(msg):
        if args.verbose:
            print(f"[bench rank {rank}] {msg}", file=sys.stderr, flush=True)

    if p > 1:
        import datetime

        # a collective that cannot complete ends the run with an error instead of hanging it
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))
    capi.lib()
    log("process group up")
    m = args.m
    n_layers = args.layers
    layers = build_layers(torch, capi, quant, p, rank, n_layers, device, m)
    log("layers built")
    ws = capi.Workspace(layers[0]["qkv"].workspace_bytes(m), device)

    bf = dict(dtype=torch.bfloat16, device=device)
    # activations are replicated under tensor parallelism: the same seed on every rank
    gen = torch.Generator(device=device).manual_seed(20240607)
    hidden = torch.randn((m, HIDDEN), generator=gen, **bf)
    resid = torch.randn((m, HIDDEN), generator=gen, **bf)
    attn_in = torch.randn((m, HIDDEN), generator=gen, **bf)            # what attention would hand to o_proj
    qkv_local = torch.empty((m, QKV_N // p), **bf)
    qkv_full = torch.empty((p, m, QKV_N // p), **bf) if p > 1 else None
    act_local = torch.empty((m, FFN // p), **bf)
    act_full = torch.empty((p, m, FFN // p), **bf) if p > 1 else None
    o_out = torch.empty((m, HIDDEN), **bf)
    d_out = torch.empty((m, HIDDEN), **bf)
    attn_slice = attn_in[:, rank * (HIDDEN // p):(rank + 1) * (HIDDEN // p)]

    launches_per_step = [0]
    # With more than one GPU the exchange is part of the linear kernels' epilogue (stores into the
    # peers' buffers over NVLink); `--collective nccl` runs the NCCL collectives after the
    # kernels instead, for comparison.
    # "auto": the fused exchange up to FUSED_MAX_TOKENS tokens, NCCL above (measured at two GPUs:
    # the fused step wins by 28 % at one token and by 8 % at eight, and loses by 13 % at sixteen,
    # where the epilogue warp's per-tile wait for the peer outweighs the saved collective
    # launches).
    want_fused = args.collective == "fused" or (args.collective == "auto" and m <= FUSED_MAX_TOKENS)
    fused = p > 1 and want_fused and m <= 16
    comm = None
    if fused:
        act_off = (m * QKV_N * 2 + 255) // 256 * 256
        comm = capi.Comm(rank, p, max(HIDDEN, 2 * FFN // p, QKV_N // p), act_off + m * FFN * 2, device)

    def step(x):
        n_launch = 0
        for L in layers:
            if fused:
                L["qkv"].linear_allgather(comm, x, gather_offset=0, workspace=ws)
                L["o_proj"].linear_allreduce(comm, attn_slice, capi.FUSE_ADD, [resid], out=o_out, workspace=ws)
                L["gate_up"].linear_allgather(comm, o_out, capi.FUSE_SILU_MUL, gather_offset=act_off, workspace=ws)
                # the row-parallel layer reads this rank's own block of the gathered activation
                act_mine = comm.gathered(act_off, m, FFN)[:, rank * (FFN // p):(rank + 1) * (FFN // p)]
                L["down_proj"].linear_allreduce(comm, act_mine, capi.FUSE_ADD, [resid], out=d_out, workspace=ws)
                n_launch += 4
                continue
            L["qkv"].linear(x, out=qkv_local, workspace=ws)
            if p > 1:
                dist.all_gather_into_tensor(qkv_full, qkv_local)
            if p == 1:
                L["o_proj"].linear(attn_slice, capi.FUSE_ADD, [resid], out=o_out, workspace=ws)
            else:
                L["o_proj"].linear(attn_slice, out=o_out, workspace=ws)
                dist.all_reduce(o_out)
                o_out.add_(resid)
            L["gate_up"].linear(o_out, capi.FUSE_SILU_MUL, out=act_local, workspace=ws)
            if p > 1:
                dist.all_gather_into_tensor(act_full, act_local)
            if p == 1:
                L["down_proj"].linear(act_local, capi.FUSE_ADD, [resid], out=d_out, workspace=ws)
            else:
                L["down_proj"].linear(act_local, out=d_out, workspace=ws)
                dist.all_reduce(d_out)
                d_out.add_(resid)
            n_launch += 4
        launches_per_step[0] = n_launch
        return d_out

    # eager warm-up (also initialises NCCL), then capture one step in a CUDA graph
    launches_before = capi.kernel_launches()
    if p > 1:
        torch.cuda.synchronize()
        dist.barrier()  # the fused exchange waits about 2 s for a peer, not for its set-up
    step(hidden)
    torch.cuda.synchronize()
    # kernels this library really launched for one step (a linear above 256 tokens is several)
    launched_per_step = capi.kernel_launches() - launches_before
    log("eager step done")
    check = None if args.no_check else verify_step(torch, dist, capi, layers[-1], p, rank, m, ws, hidden, resid,
                                                     attn_slice, fused, comm, act_off if fused else 0,
                                                     qkv_local if p == 1 else (None if fused else qkv_full),
                                                     o_out, act_local if p == 1 else (None if fused else act_full),
                                                     d_out)
    log(f"outputs checked: {check}")
    graph = None
    if not args.no_graph:
        try:
            side = torch.cuda.Stream(device=device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(hidden)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step(hidden)
        except Exception as e:  # pragma: no cover - depends on the NCCL build
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); running eagerly",
                      file=sys.stderr)
            graph = None
            torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step(hidden)

    def barrier():
        if p > 1:
            dist.barrier()
        torch.cuda.synchronize()

    log(f"graph captured: {graph is not None}")
    for _ in range(max(3, args.warmup)):
        run_step()
    barrier()
    log("warm-up done")
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    if p > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    log(f"timed region done: {ms_per_step:.3f} ms/step")
    total_w = full_layer_weight_bytes() * n_layers  # all ranks together stream the whole model
    value = total_w / (ms_per_step * 1e-3) / 1e9
    ws.status()

    # ---- kernel-only timing for the roofline (linears alone, no collectives) --------------
    def linears_only():
        for L in layers:
            L["qkv"].linear(hidden, out=qkv_local, workspace=ws)
            L["o_proj"].linear(attn_slice, capi.FUSE_ADD if p == 1 else 0, [resid] if p == 1 else [],
                               out=o_out, workspace=ws)
            L["gate_up"].linear(o_out, capi.FUSE_SILU_MUL, out=act_local, workspace=ws)
            L["down_proj"].linear(act_local, capi.FUSE_ADD if p == 1 else 0, [resid] if p == 1 else [],
                                  out=d_out, workspace=ws)

    kgraph = torch.cuda.CUDAGraph()
    linears_only()
    torch.cuda.synchronize()
    with torch.cuda.graph(kgraph):
        linears_only()
    for _ in range(3):
        kgraph.replay()
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(3, min(args.steps, 10))
    k0.record()
    for _ in range(reps):
        kgraph.replay()
    k1.record()
    torch.cuda.synchronize()
    n_launch = launches_per_step[0]
    kernel_ms = k0.elapsed_time(k1) / reps / n_launch
    local_bytes = sum(weight_bytes(n, k) + 2 * m * k + 2 * m * (n // 2 if name == "gate_up" else n)
                      + (2 * m * n if (p == 1 and kind == "row") else 0)
                      for name, n, k, kind in layer_shapes(p)) * n_layers
    hbm_peak, tf_peak_r, peak_src = peaks()
    achieved = local_bytes / n_launch / (kernel_ms * 1e-3) / 1e9
    if m > 16:
        # above decode sizes the linears are contractions on the tensor cores
        flops = sum(2.0 * m * n * k for _, n, k, _ in layer_shapes(p)) * n_layers
        tf = flops / n_launch / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": tf, "peak": tf_peak_r, "unit": "TFLOP/s",
                    "frac": tf / tf_peak_r if tf_peak_r else None, "traffic": None,
                    "kernel": "woq_int4_tc_kernel", "peak_source": peak_src, "avg_launch_us": kernel_ms * 1e3,
                    "algorithmic_flops_per_launch": flops / n_launch}
    else:
        roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": achieved / hbm_peak,
                    "traffic": args.traffic if args.traffic is not None else TRAFFIC_RATIO * local_bytes / n_launch,
                    "kernel": "woq_int4_decode_kernel", "peak_source": peak_src,
                    "avg_launch_us": kernel_ms * 1e3,
                    "algorithmic_bytes_per_launch": local_bytes / n_launch}

    # ---- end to end: host activations in, host result out, through the module API ---------
    x_host = torch.randn((m, HIDDEN)).bfloat16().pin_memory()
    y_host = torch.empty((m, HIDDEN), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        hidden.copy_(x_host, non_blocking=True)
        run_step()
        y_host.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    if p > 1:
        t = torch.tensor([e2e_s], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": total_w / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": m * HIDDEN * 2,
           "d2h_bytes_per_step": m * HIDDEN * 2, "ms_per_step": e2e_s * 1e3}

    e2e_ops = None
    if p == 1 and m <= 16 and not args.no_e2e_ops:
        e2e_ops = e2e_through_ops(torch, quant, m, device)
        log(f"e2e through the ops: {e2e_ops}")

    # ---- prefill side of the metric: the tcgen05 kernel on one gate_up-sized layer ----------
    prefill = None
    if p == 1 and not args.no_prefill:
        pm = 512
        g = torch.Generator(device=device).manual_seed(4242)
        w = torch.randn((2 * FFN, HIDDEN), device=device, generator=g) * 0.02
        qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
        del w
        pctx = [capi.WoqContext(qw, s.half(), z, None, 2 * FFN, HIDDEN, capi.DTYPE_INT4, GROUP, capi.LOWP_BF16,
                                layout_flags=capi.LAYOUT_TC_ONLY) for _ in range(2)]
        del qw, s, z
        px = torch.randn((pm, HIDDEN), **bf)
        py = torch.empty((pm, 2 * FFN), **bf)
        pws = capi.Workspace(pctx[0].workspace_bytes(pm), device)
        for c in pctx:
            c.linear(px, out=py, workspace=pws)
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        preps = 6
        p0.record()
        for i in range(preps):
            pctx[i % 2].linear(px, out=py, workspace=pws)
        p1.record()
        torch.cuda.synchronize()
        pws.status()
        pt = p0.elapsed_time(p1) * 1e-3 / preps
        _, tf_peak, _ = peaks()
        tflops = 2.0 * pm * 2 * FFN * HIDDEN / pt / 1e12
        prefill = {"tflops": tflops, "m": pm, "shape": f"{2 * FFN}x{HIDDEN} INT4 g128", "us_per_linear": pt * 1e6,
                   "kernel": "woq_int4_tc_kernel", "bound": "tensor", "peak": tf_peak, "unit": "TFLOP/s",
                   "frac": tflops / tf_peak if tf_peak else None}
        del pctx, px, py, pws

    # ---- side line: the scale-after-sum dequantiser (WOQ_B200_HINT_STREAM_FAST) on one layer's
    # four shapes beside the per-weight default, with the deviation between the two --------------
    stream_fast = None
    if p == 1 and m <= 8 and not args.no_fast:
        stream_fast = fast_side_line(torch, capi, quant, device, m)
        log(f"scale-after-sum side line: {stream_fast}")

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": p, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3-70b linears (QKV 10240x8192, o 8192x8192, gate_up 57344x8192 "
                                   "silu_mul, down 8192x28672), INT4 asym g128, lowp BF16, decode",
                       "m": m, "layers": n_layers, "parallelism": f"tp{p}",
                       "collective": ("none" if p == 1 else "fused into the linear kernels (peer stores over NVLink)"
                                      if fused else "nccl"),
                       "l2": f"weights ({total_w / 1e9:.1f} GB per step over all ranks) exceed L2; no flush needed",
                       "cuda_graph": graph is not None},
            "roofline": roofline, "prefill": prefill, "stream_fast": stream_fast, "e2e": e2e, "e2e_ops": e2e_ops,
            "checked": check is not None, "check": check, "gpu_launches": launched_per_step * args.steps,
            "clocks": clocks,
        }
        if p == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(m)
        print(json.dumps(line), flush=True)
    if p > 1:
        # Tearing down NCCL communicators that were captured into CUDA graphs can block for
        # minutes; every rank has its result by now, so leave without the teardown.
        del graph, kgraph
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_single(args):
    """A few launches of one linear shape (for `ncu` captures of a small case):
    --single NxK --m M [--hint H] launches the linear `--steps` times on two weight copies."""
    import torch

    from ipex_b200 import _capi as capi
    from ipex_b200 import quantization as quant

    n, k = (int(v) for v in args.single.lower().split("x"))
    torch.cuda.set_device(0)
    ctxs = []
    for i in range(2):
        g = torch.Generator(device="cuda").manual_seed(i)
        w = torch.randn((n, k), device="cuda", generator=g) * 0.02
        if args.int8:
            qw, s, _ = quant.quantize_per_channel(w, quant.WoqWeightDtype.INT8, sym_quant=True)
            ctxs.append(capi.WoqContext(qw, s, None, None, n, k, capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                                        act_quant_mode=capi.ACT_PER_M_SYM))
        else:
            qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
            ctxs.append(capi.WoqContext(qw, s.half(), z, None, n, k, capi.DTYPE_INT4, GROUP, capi.LOWP_BF16,
                                        kernel_hint=args.hint))
    x = torch.randn((args.m, k), device="cuda").bfloat16()
    y = torch.empty((args.m, n), device="cuda", dtype=torch.bfloat16)
    ws = capi.Workspace(ctxs[0].workspace_bytes(args.m), "cuda")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for c in ctxs:
        c.linear(x, out=y, workspace=ws)
    e0.record()
    for _ in range(args.steps):
        for c in ctxs:
            c.linear(x, out=y, workspace=ws)
    e1.record()
    torch.cuda.synchronize()
    ws.status()
    us = e0.elapsed_time(e1) * 1e3 / (2 * args.steps)
    print(json.dumps({"single": args.single, "m": args.m, "int8": args.int8, "hint": args.hint,
                      "us_per_launch": us, "weight_GBps": (n * k if args.int8 else weight_bytes(n, k)) / us / 1e3,
                      "tflops": 2 * args.m * n * k / us / 1e6}))


# ------------------------------------------------------------------------------------------
# --configs: every benchmark configuration's linear shapes, one JSON line per case
# ------------------------------------------------------------------------------------------
# (config, name, N, K, weights, fused epilogue, token counts)
CONFIG_CASES = [
    ("c1-single-int4", "linear", 4096, 4096, "int4", "none", (1, 4, 32, 256)),
    ("c2-llama3-8b-int8", "qkv", 6144, 4096, "int8", "none", (1, 8, 64, 512)),
    ("c2-llama3-8b-int8", "o_proj", 4096, 4096, "int8", "none", (1, 8, 64, 512)),
    ("c2-llama3-8b-int8", "gate_up", 28672, 4096, "int8", "silu_mul", (1, 8, 64, 512)),
    ("c2-llama3-8b-int8", "down_proj", 4096, 14336, "int8", "add", (1, 8, 64, 512)),
    ("c3-llama3-8b-int4", "qkv", 6144, 4096, "int4", "none", (1, 8, 32, 1024)),
    ("c3-llama3-8b-int4", "o_proj", 4096, 4096, "int4", "add", (1, 8, 32, 1024)),
    ("c3-llama3-8b-int4", "gate_up", 28672, 4096, "int4", "silu_mul", (1, 8, 32, 1024)),
    ("c3-llama3-8b-int4", "down_proj", 4096, 14336, "int4", "add", (1, 8, 32, 1024)),
    ("c5-llama3-70b-int4", "qkv", 10240, 8192, "int4", "none", (1, 16, 128)),
    ("c5-llama3-70b-int4", "o_proj", 8192, 8192, "int4", "add", (1, 16, 128)),
    ("c5-llama3-70b-int4", "gate_up", 57344, 8192, "int4", "silu_mul", (1, 16, 128)),
    ("c5-llama3-70b-int4", "down_proj", 8192, 28672, "int4", "add", (1, 16, 128)),
]
MOE_TOKENS = (1, 16, 256, 4096)  # c4: 8 experts, top-2, w13 28672x4096 silu_mul, w2 4096x14336 scaled add
ROTATE_BYTES = 300e6             # weight copies walked per pass: more than twice the L2


def _time_graph(torch, fn, launches_per_pass, min_ms=40.0):
    """Median over five timed blocks of graph replays of `fn`; returns microseconds per launch."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        graph.replay()
        e1.record(stream)
        stream.synchronize()
        reps = max(3, min(200, int(min_ms / 5 / max(e0.elapsed_time(e1), 1e-3))))
        samples = []
        for _ in range(5):
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            samples.append(e0.elapsed_time(e1) / reps)
    return statistics.median(samples) * 1e3 / launches_per_pass


def run_configs(args):
    """Every configuration's linears at its token counts on one GPU: CUDA-graph replay over
    rotating weight copies (more than twice the L2), CUDA events, median of five blocks.  One
    JSON line per case: time, weight and total GB/s, TFLOP/s and the fraction of the bound that
    applies (HBM below the ridge point, tensor above; INT8 against twice the bf16 peak)."""
    import torch

    from ipex_b200 import _capi as capi
    from ipex_b200 import quantization as quant

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    hbm, tf, which = peaks()
    only = args.configs if args.configs != "all" else None

    def make_ctx(n, k, kind, fusion, m, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        w = torch.randn((n, k), device=dev, generator=g) * 0.02
        gate_up = capi.LAYOUT_GATE_UP if fusion == "silu_mul" else 0
        if kind == "int8":
            qw, s, _ = quant.quantize_per_channel(w, quant.WoqWeightDtype.INT8, sym_quant=True)
            return capi.WoqContext(qw, s, None, None, n, k, capi.DTYPE_INT8, -1, capi.LOWP_INT8,
                                   act_quant_mode=capi.ACT_PER_M_SYM, layout_flags=gate_up)
        qw, s, z = quant.quantize_per_block(w, quant.WoqWeightDtype.INT4, GROUP)
        tiling = capi.LAYOUT_STREAM_ONLY if m <= 16 else capi.LAYOUT_TC_ONLY
        return capi.WoqContext(qw, s.half(), z, None, n, k, capi.DTYPE_INT4, GROUP, capi.LOWP_BF16,
                               layout_flags=tiling | gate_up, kernel_hint=args.hint if m <= 16 else 0)

    def report(config, name, n, k, kind, fusion, m, us, wbytes, total, flops, note=None):
        ai = flops / total
        peak_tf = tf * (2.0 if kind == "int8" else 1.0)
        bound = "tensor" if ai > peak_tf * 1e3 / hbm else "hbm"
        frac = (flops / us / 1e6) / peak_tf if bound == "tensor" else (total / us / 1e3) / hbm
        line = {"config": config, "linear": name, "n": n, "k": k, "weights": kind, "fusion": fusion, "m": m,
                "hint": args.hint, "split": args.split,
                "us": round(us, 2), "weight_GBps": round(wbytes / us / 1e3, 1),
                "total_GBps": round(total / us / 1e3, 1), "tflops": round(flops / us / 1e6, 2),
                "bound": bound, "frac_of_" + which: round(frac, 3)}
        if note:
            line["note"] = note
        print(json.dumps(line), flush=True)

    for config, name, n, k, kind, fusion, ms in CONFIG_CASES:
        if only and not config.startswith(only):
            continue
        wbytes = n * k + 4 * n if kind == "int8" else weight_bytes(n, k)
        copies = max(2, min(40, int(ROTATE_BYTES // wbytes) + 1))
        fuse = {"none": capi.FUSE_NONE, "silu_mul": capi.FUSE_SILU_MUL, "add": capi.FUSE_ADD}[fusion]
        n_out = n // 2 if fusion == "silu_mul" else n
        ctxs, tiling_m = [], None
        for m in ms:
            if m > args.max_m:
                continue
            if kind == "int8" or tiling_m is None or (tiling_m <= 16) != (m <= 16):
                for c in ctxs:
                    c.close()
                ctxs = [make_ctx(n, k, kind, fusion, m, 7 * i + 1) for i in range(copies)]
                tiling_m = m
            x = torch.randn((m, k), device=dev).bfloat16()
            y = torch.empty((m, n_out), device=dev, dtype=torch.bfloat16)
            others = [torch.randn((m, n_out), device=dev).bfloat16()] if fusion == "add" else []
            ws = capi.Workspace(ctxs[0].workspace_bytes(m), dev)

            def one_pass():
                for c in ctxs:
                    c.linear(x, fuse, others, out=y, workspace=ws)

            us = _time_graph(torch, one_pass, copies)
            ws.status()
            total = wbytes + 2 * m * k + 2 * m * n_out * (1 + len(others))
            report(config, name, n, k, kind, fusion, m, us, wbytes, total, 2.0 * m * n * k)
        for c in ctxs:
            c.close()
        del ctxs
        torch.cuda.empty_cache()

    if only and not "c4-mixtral-moe".startswith(only):
        return
    # c4: one sparse-MoE layer, experts replicated on this GPU, top-2 routing from seeded logits
    hid, ffn, n_exp = 4096, 14336, 8
    experts = []
    for e in range(n_exp):
        experts.append((make_ctx(2 * ffn, hid, "int4", "silu_mul", 1, 100 + e), make_ctx(hid, ffn, "int4", "none", 1, 200 + e)))
    for t in MOE_TOKENS:
        if t > args.max_m:
            continue
        if t > 16:  # the expert linears switch tiling with the token count
            for a, b in experts:
                a.close()
                b.close()
            experts = [(make_ctx(2 * ffn, hid, "int4", "silu_mul", t, 100 + e), make_ctx(hid, ffn, "int4", "none", t, 200 + e))
                       for e in range(n_exp)]
        g = torch.Generator(device=dev).manual_seed(4000 + t)
        hidden = torch.randn((t, hid), device=dev, generator=g).bfloat16()
        router = torch.randn((n_exp, hid), device=dev, generator=g) * 0.02
        prob = torch.softmax(hidden.float() @ router.t(), dim=-1)
        top_w, top_e = prob.topk(2, dim=-1)
        top_w = (top_w / top_w.sum(-1, keepdim=True)).bfloat16()
        plan = []
        for e in range(n_exp):
            tok, slot = (top_e == e).nonzero(as_tuple=True)
            if tok.numel():
                plan.append((e, tok.int().contiguous(), top_w[tok, slot].contiguous()))
        out = torch.zeros((t, hid), device=dev, dtype=torch.bfloat16)
        wss = {e: capi.moe_expert(experts[e][0], experts[e][1], hidden, idx, w, out) for e, idx, w in plan}

        def one_layer():
            for e, idx, w in plan:
                capi.moe_expert(experts[e][0], experts[e][1], hidden, idx, w, out, workspace=wss[e])

        us = _time_graph(torch, one_layer, 1)
        for w_ in wss.values():
            w_.status()
        wbytes = len(plan) * (weight_bytes(2 * ffn, hid) + weight_bytes(hid, ffn))
        assigned = sum(int(idx.numel()) for _, idx, _ in plan)
        total = wbytes + assigned * (2 * hid + 2 * ffn * 2 + 2 * hid * 2)
        flops = 2.0 * assigned * (2 * ffn * hid + hid * ffn)
        report("c4-mixtral-moe", "layer (8 experts, top-2)", 2 * ffn, hid, "int4", "silu_mul + scaled add", t, us,
               wbytes, total, flops, note=f"{len(plan)} experts active, {assigned} token assignments, one layer per pass "
               f"(weights {'above' if wbytes > 2.5e8 else 'below'} twice the L2)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", "--tokens", dest="m", type=int, default=1,
                    help="decode batch (tokens per step); spell it --tokens under torch.distributed.run")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="phase messages on stderr")
    ap.add_argument("--collective", default="auto", choices=["auto", "fused", "nccl"],
                    help="N > 1: exchange inside the linear kernels, NCCL after them, or (auto) the "
                         "fused exchange up to %d tokens" % FUSED_MAX_TOKENS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the check of the step's outputs before timing")
    ap.add_argument("--no-e2e-ops", action="store_true", help="skip the end-to-end leg through torch.ops")
    ap.add_argument("--no-fast", action="store_true", help="skip the scale-after-sum side line")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill (tensor-core kernel) side line")
    ap.add_argument("--single", default=None, help="NxK: run one linear shape only (profiler captures)")
    ap.add_argument("--int8", action="store_true", help="--single: INT8 weights with INT8 compute")
    ap.add_argument("--hint", type=int, default=0, help="--single: kernel hint (see include/woq_b200.h)")
    ap.add_argument("--max-m", type=int, default=1 << 30, help="--configs: skip token counts above this")
    ap.add_argument("--split", type=int, default=None, choices=[0, 1, 2],
                    help="decode kernel's K split: 0 per layer, 1 stream-K, 2 clusters (woq_b200_set_option)")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch from an ncu capture (default: TRAFFIC_RATIO x algorithmic bytes)")
    ap.add_argument("--configs", default=None, nargs="?", const="all",
                    help="time every benchmark configuration's linears (optionally a prefix: c1, c2, c3, c4, c5)")
    ap.add_argument("--stack", default=None, nargs="?", const="all",
                    help="the Llama-3-8B-architecture decode stack (bench_stack.py); optionally batch sizes, e.g. 1,8")
    ap.add_argument("--new-tokens", type=int, default=128, help="--stack: greedy decode steps")
    args = ap.parse_args()
    if args.split is not None:
        from ipex_b200 import _capi

        _capi.set_option(_capi.OPT_DECODE_SPLIT, args.split)
    if args.stack:
        import bench_stack

        bench_stack.run_stack(args, peaks, ClockSampler)
    elif args.configs:
        run_configs(args)
    elif args.single:
        run_single(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
