"""Generate the golden fixtures in this folder from the reference tree.

Run once, in a container where the reference project is checked out, as

    python tests/golden/make_golden.py /path/to/intel-extension-for-pytorch

The reference package itself cannot be imported (it needs its compiled extension), but the
pieces that pin the WOQ linear path are plain PyTorch and are executed here as text:

  * the weight quantiser / dequantiser
    (intel_extension_for_pytorch/quantization/_quantize_utils.py, from NF4_QUANT_TABLE to
    the end of the file) together with the WoqWeightDtype enum
    (intel_extension_for_pytorch/quantization/_qconfig.py);
  * dequantize_awq and its helper from tests/cpu/test_ipex_llm_quantization.py, applied to
    the known-answer tensors tests/cpu/data/awq/*.pt;
  * the activation fake-quantisers _fakequant_by_group / _fakequant_by_group_sym from
    tests/cpu/test_quantization_default_recipe.py (all eight activation quantisation modes).

Outputs (inputs and the reference's results, nothing else):
  quantizer_cases.npz   seeded weights -> qweight / scales / zero points / dequantised
  awq_fixture.npz       AWQ checkpoint tensors, a slice of the activation, and the
                        reference-dequantised bf16 weight and reference output
  act_quant_cases.npz   seeded activations -> reference fake-quantised activations
  act_quant_modes.npz   the same for every activation quantisation mode (0..7), K-block 128
"""
import os
import re
import sys
import textwrap
from enum import IntEnum
from typing import Optional

import numpy as np
import torch


def _load_quantizer(ref):
    src = open(
        os.path.join(ref, "intel_extension_for_pytorch/quantization/_quantize_utils.py")
    ).read()
    start = src.index("NF4_QUANT_TABLE = [")
    qc = open(os.path.join(ref, "intel_extension_for_pytorch/quantization/_qconfig.py")).read()
    m = re.search(r"class WoqWeightDtype\(IntEnum\):\n(?:    .*\n)+", qc)
    ns = {"torch": torch, "Optional": Optional, "IntEnum": IntEnum, "__name__": "ref_quant"}
    exec(m.group(0), ns)
    exec(src[start:], ns)
    return ns


def _load_awq_helpers(ref):
    src = open(os.path.join(ref, "tests/cpu/test_ipex_llm_quantization.py")).read()
    a = src.index("def awq_reverse_reorder_int_tensor")
    b = src.index("class TestLLMQuantization")
    ns = {"torch": torch}
    exec(src[a:b], ns)
    return ns


def _load_fakequant(ref, asym=False):
    src = open(os.path.join(ref, "tests/cpu/test_quantization_default_recipe.py")).read()
    a = src.index("    def _fakequant_by_group(" if asym else "    def _fakequant_by_group_sym(")
    b = src.index("    def test_weight_only_quantization_act_quant_mode(")
    ns = {"torch": torch}
    exec(textwrap.dedent(src[a:b]), ns)
    return ns["_fakequant_by_group" if asym else "_fakequant_by_group_sym"]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().bfloat16().contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref):
    here = os.path.dirname(os.path.abspath(__file__))
    q = _load_quantizer(ref)
    W = q["WoqWeightDtype"]

    # ---- quantiser cases ------------------------------------------------------------
    cases = {}
    specs = [
        # name, N, K, dtype, group, sym, std
        ("int4_g128_asym", 48, 512, W.INT4, 128, False, 0.02),
        ("int4_g64_asym", 40, 256, W.INT4, 64, False, 0.02),
        ("int4_g32_sym", 33, 160, W.INT4, 32, True, 0.05),
        ("int4_g128_rem", 24, 320, W.INT4, 128, False, 0.02),
        ("int4_pc_asym", 32, 200, W.INT4, -1, False, 0.02),
        ("int8_pc_sym", 64, 384, W.INT8, -1, True, 0.02),
        ("int8_g128_asym", 32, 256, W.INT8, 128, False, 0.02),
        ("nf4_g64_sym", 24, 256, W.NF4, 64, True, 0.02),
        ("nf4_pc_sym", 16, 200, W.NF4, -1, True, 0.05),
    ]
    for i, (name, N, K, dt, G, sym, std) in enumerate(specs):
        torch.manual_seed(100 + i)
        w = torch.randn(N, K) * std
        if i == 0:
            w[3] = 0.0  # an all-zero row: scale clamps to fp32 eps
            w[5, :128] = w[5, :128].abs()  # a group with min clamped to 0
        if G > 0:
            qw, s, z = q["quantize_per_block"](w, dt, G, None, None, sym)
            dq = q["dequantize_per_block"](qw, s, z, dt, G, [N, K])
        else:
            qw, s, z = q["quantize_per_channel"](w, dt, None, None, sym)
            dq = q["dequantize_per_channel"](qw, s, z, dt, [N, K])
        cases[name + ".w"] = w.numpy()
        cases[name + ".qw"] = qw.numpy()
        cases[name + ".scales"] = s.numpy()
        if z is not None:
            cases[name + ".zps"] = z.numpy()
        cases[name + ".dq"] = dq.numpy()
        cases[name + ".meta"] = np.array([N, K, int(dt), G, int(sym)], dtype=np.int64)
    np.savez_compressed(os.path.join(here, "quantizer_cases.npz"), **cases)

    # ---- AWQ known-answer tensors -----------------------------------------------------
    a = _load_awq_helpers(ref)
    d = os.path.join(ref, "tests/cpu/data/awq")
    qweight = torch.load(os.path.join(d, "qweight.pt"), weights_only=True)
    qzeros = torch.load(os.path.join(d, "qzeros.pt"), weights_only=True)
    scales = torch.load(os.path.join(d, "scales.pt"), weights_only=True)
    bias = torch.load(os.path.join(d, "bias.pt"), weights_only=True)
    act = torch.load(os.path.join(d, "act.pt"), weights_only=True)
    w_ref = a["dequantize_awq"](qweight, qzeros, scales, 4, 128)  # [N, K] bf16
    rows = torch.arange(0, act.shape[0], 29)[:24]  # 24 of the 677 activation rows
    act_s = act[rows].contiguous()
    y_ref = torch.matmul(act_s, w_ref.T) + bias
    np.savez_compressed(
        os.path.join(here, "awq_fixture.npz"),
        qweight=qweight.numpy(),
        qzeros=qzeros.numpy(),
        scales_bf16=bf16_bits(scales),
        bias_bf16=bf16_bits(bias),
        act_bf16=bf16_bits(act_s),
        act_rows=rows.numpy(),
        w_ref_rows=np.arange(0, w_ref.shape[0], 4),
        w_ref_bf16=bf16_bits(w_ref[::4].contiguous()),  # every 4th output channel
        y_ref_bf16=bf16_bits(y_ref),
        group_size=np.int64(128),
    )

    # ---- activation fake-quant (per token, symmetric) ---------------------------------
    fq = _load_fakequant(ref)
    acts = {}
    for i, (M, K) in enumerate([(5, 256), (16, 512), (3, 4096)]):
        torch.manual_seed(200 + i)
        x = torch.randn(M, K).bfloat16()
        # mode 6 = PER_BATCH_SYM, one group per row.  The bf16 values are handed over as
        # float32 so that the helper's arithmetic (max/127, true division, round half to
        # even) runs in fp32 like the kernel it models; with a bf16 tensor it would round
        # the scale to bf16 first.
        out = fq(None, x.float(), 6, K)
        acts[f"c{i}.x_bf16"] = bf16_bits(x)
        acts[f"c{i}.fq_f32"] = out.numpy()
    np.savez_compressed(os.path.join(here, "act_quant_cases.npz"), **acts)

    # ---- every activation quantisation mode: 0 per tensor, 1 per K block, 2 per token, 3 per
    # token and K block; +4 symmetric (csrc/cpu/aten/utils/woq_defines.h:11-19) ----------
    fq_asym = _load_fakequant(ref, asym=True)
    modes = {}
    for i, (M, K) in enumerate([(4, 256), (9, 384), (2, 1024)]):
        torch.manual_seed(300 + i)
        x = (torch.randn(M, K) + 0.3).bfloat16()  # a range that is not centred on zero
        modes[f"c{i}.x_bf16"] = bf16_bits(x)
        for mode in range(8):
            out = (fq_asym if mode < 4 else fq)(None, x.float(), mode, 128)
            modes[f"c{i}.mode{mode}_f32"] = out.numpy()
    np.savez_compressed(os.path.join(here, "act_quant_modes.npz"), **modes)
    print("golden fixtures written to", here)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of intel-extension-for-pytorch>")
    main(sys.argv[1])
