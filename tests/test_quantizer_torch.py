"""The package's torch quantiser must reproduce the reference quantiser's golden outputs."""
import os

import numpy as np
import pytest
import torch

from ipex_b200.quantization import (WoqWeightDtype, dequantize_per_block, dequantize_per_channel,
                                    get_weight_only_quant_qconfig_mapping, quantize_per_block,
                                    quantize_per_channel, WoqLowpMode, WoqActQuantMode, WoqWeightQScheme)

CASES = ["int4_g128_asym", "int4_g64_asym", "int4_g32_sym", "int4_g128_rem", "int4_pc_asym",
         "int8_pc_sym", "int8_g128_asym"]


@pytest.mark.parametrize("name", CASES)
def test_against_reference_golden(golden_dir, name):
    f = np.load(os.path.join(golden_dir, "quantizer_cases.npz"))
    N, K, dt, G, sym = (int(v) for v in f[name + ".meta"])
    w = torch.from_numpy(f[name + ".w"])
    if G > 0:
        qw, s, z = quantize_per_block(w, dt, G, sym_quant=bool(sym))
        dq = dequantize_per_block(qw, s, z, dt, G, [N, K])
    else:
        qw, s, z = quantize_per_channel(w, dt, sym_quant=bool(sym))
        dq = dequantize_per_channel(qw, s, z, dt, [N, K])
    np.testing.assert_array_equal(qw.numpy(), f[name + ".qw"])
    np.testing.assert_array_equal(s.numpy().view(np.uint32), f[name + ".scales"].view(np.uint32))
    if not sym:
        np.testing.assert_array_equal(z.numpy(), f[name + ".zps"])
    np.testing.assert_array_equal(dq.numpy(), f[name + ".dq"])


def test_qconfig_defaults_and_rules():
    m = get_weight_only_quant_qconfig_mapping()
    q = m.global_qconfig
    assert q.weight_dtype == WoqWeightDtype.INT8 and q.lowp_mode == WoqLowpMode.NONE
    assert q.act_quant_mode == WoqActQuantMode.NONE and q.group_size == -1
    assert q.weight_qscheme == WoqWeightQScheme.ASYMMETRIC
    q = get_weight_only_quant_qconfig_mapping(weight_dtype=WoqWeightDtype.INT8,
                                              lowp_mode=WoqLowpMode.INT8).global_qconfig
    assert q.weight_qscheme == WoqWeightQScheme.SYMMETRIC
    assert q.act_quant_mode == WoqActQuantMode.PER_BATCH_IC_BLOCK_SYM
    with pytest.raises(AssertionError):
        get_weight_only_quant_qconfig_mapping(group_size=48)
    with pytest.raises(AssertionError):
        get_weight_only_quant_qconfig_mapping(weight_dtype=WoqWeightDtype.INT8, lowp_mode=WoqLowpMode.INT8,
                                              weight_qscheme=WoqWeightQScheme.ASYMMETRIC)
