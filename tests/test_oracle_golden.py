"""Pins the CPU oracle against results produced by the reference's own Python code
(tests/golden/make_golden.py says how each fixture was made)."""
import os

import numpy as np
import pytest

from oracle import woq_oracle as O

QUANT_CASES = [
    "int4_g128_asym",
    "int4_g64_asym",
    "int4_g32_sym",
    "int4_g128_rem",
    "int4_pc_asym",
    "int8_pc_sym",
    "int8_g128_asym",
    "nf4_g64_sym",
    "nf4_pc_sym",
]


@pytest.fixture(scope="module")
def qcases(golden_dir):
    return np.load(os.path.join(golden_dir, "quantizer_cases.npz"))


@pytest.mark.parametrize("name", QUANT_CASES)
def test_quantizer_bit_exact(qcases, name):
    N, K, dt, G, sym = (int(v) for v in qcases[name + ".meta"])
    w = qcases[name + ".w"]
    if G > 0:
        qw, s, z = O.quantize_per_block(w, dt, G, bool(sym))
    else:
        qw, s, z = O.quantize_per_channel(w, dt, bool(sym))
    ref_qw = qcases[name + ".qw"]
    assert qw.dtype == ref_qw.dtype and qw.shape == ref_qw.shape
    np.testing.assert_array_equal(qw, ref_qw)
    np.testing.assert_array_equal(s.view(np.uint32), qcases[name + ".scales"].view(np.uint32))
    if sym:
        assert z is None and (name + ".zps") not in qcases
    else:
        np.testing.assert_array_equal(z, qcases[name + ".zps"])


@pytest.mark.parametrize("name", QUANT_CASES)
def test_dequantizer_matches_reference_fp32(qcases, name):
    """scale_rounding='none' without output rounding is the reference's fp32 dequantiser."""
    N, K, dt, G, sym = (int(v) for v in qcases[name + ".meta"])
    zps = None if sym else qcases[name + ".zps"]
    dq = O.dequantize_weight(
        qcases[name + ".qw"], qcases[name + ".scales"], zps, dt, K, G,
        scale_rounding="none", round_output=False,
    )
    np.testing.assert_array_equal(dq.view(np.uint32), qcases[name + ".dq"].view(np.uint32))


def test_canonical_dequant_is_bf16_of_bf16_scale(qcases):
    name = "int4_g128_asym"
    N, K, dt, G, sym = (int(v) for v in qcases[name + ".meta"])
    dq = O.dequantize_weight(qcases[name + ".qw"], qcases[name + ".scales"].astype(np.float16),
                             qcases[name + ".zps"], dt, K, G)
    q = O.unpack_nibbles(qcases[name + ".qw"]).astype(np.float32)
    s = O.rne_bf16(qcases[name + ".scales"].astype(np.float16).astype(np.float32))
    z = qcases[name + ".zps"]
    expect = O.rne_bf16((q - np.repeat(z, G, 1)) * np.repeat(s, G, 1))
    np.testing.assert_array_equal(dq.view(np.uint32), expect.view(np.uint32))
    assert np.all((dq.view(np.uint32) & 0xFFFF) == 0)


def test_rne_bf16_against_torch():
    import torch

    rng = np.random.default_rng(0)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 3,
        np.array([0.0, -0.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, np.inf, -np.inf],
                 dtype=np.float32),
    ])
    ours = O.rne_bf16(x)
    ref = torch.from_numpy(x).bfloat16().float().numpy()
    np.testing.assert_array_equal(ours.view(np.uint32), ref.view(np.uint32))


def test_awq_fixture(golden_dir):
    """The reference's AWQ known-answer tensors: integer codes and zero points must come
    out exactly, the dequantised weight and the output within the reference test's own
    tolerance (tests/cpu/test_ipex_llm_quantization.py:151 uses prec=0.1)."""
    f = np.load(os.path.join(golden_dir, "awq_fixture.npz"))
    G = int(f["group_size"])
    scales = O.from_bf16_bits(f["scales_bf16"])  # [K/G, N]
    qw, s, z = O.awq_to_plain(f["qweight"], f["qzeros"], scales)
    K = f["qweight"].shape[0]
    N = f["qweight"].shape[1] * 8
    assert qw.shape == (N, K // 2) and s.shape == (N, K // G) and z.shape == (N, K // G)
    w_ref = O.from_bf16_bits(f["w_ref_bf16"])  # rows w_ref_rows of [N, K]
    rows = f["w_ref_rows"]
    # the reference test computes q*s - bf16(z*s) in bf16; ours is (q-z)*s rounded once:
    # equal up to bf16 rounding of numbers of size |q*s|.
    w = O.dequantize_weight(qw, s, z, O.WOQ_DTYPE_INT4, K, G)[rows]
    tol = np.abs(w_ref).max() * 2.0 ** -7
    assert np.abs(w - w_ref).max() <= tol
    # exact check of the integer part: recover q - z from the reference weight
    sfull = np.repeat(s[rows], G, axis=1)
    qz = O.unpack_nibbles(qw)[rows].astype(np.float32) - np.repeat(z[rows], G, axis=1)
    assert np.abs(np.rint(w_ref / sfull) - qz).max() <= 1.0
    assert (np.rint(w_ref / sfull) == qz).mean() > 0.98
    x = O.from_bf16_bits(f["act_bf16"])
    bias = O.from_bf16_bits(f["bias_bf16"])
    y = O.woq_linear_bf16(x, qw, s, z, bias, O.WOQ_DTYPE_INT4, G)
    y_ref = O.from_bf16_bits(f["y_ref_bf16"])
    assert np.abs(y - y_ref).max() <= 0.1
    mx, mr = O.parity_metrics(y, y_ref)
    assert mx < 2e-2 and mr < 1e-2


def test_act_quant_against_reference_fakequant(golden_dir):
    """Codes * scale must reproduce the reference test's per-token symmetric fake-quant
    (tests/cpu/test_quantization_default_recipe.py:915-979, mode 6)."""
    f = np.load(os.path.join(golden_dir, "act_quant_cases.npz"))
    for i in range(3):
        x = O.from_bf16_bits(f[f"c{i}.x_bf16"])
        fq_ref = f[f"c{i}.fq_f32"]
        q, s, _ = O.dynamic_quant_per_token(x, sym=True)
        fq = q.astype(np.float32) * s[:, None]
        np.testing.assert_array_equal(fq, fq_ref)  # value equality (-0.0 == 0.0)
        assert q.min() >= -128 and q.max() <= 127 and np.abs(q).max() == 127


def test_act_order_dequant_matches_a_per_element_restatement():
    """W[n][k] = bf16((q - zp[n][g_idx[k]]) * bf16(scale[n][g_idx[k]])), element by element."""
    rng = np.random.default_rng(0)
    n, k, g = 6, 256, 64
    g_idx = rng.permutation(np.arange(k) // g)
    q = rng.integers(0, 16, (n, k)).astype(np.uint8)
    qw = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    s = (rng.random((n, k // g)) * 0.01 + 0.002).astype(np.float16)
    z = rng.integers(0, 16, (n, k // g)).astype(np.float32)
    w = O.dequantize_weight_act_order(qw, s, z, g_idx, k)
    for i in range(n):
        for j in range(0, k, 7):
            sc = O.rne_bf16(np.float32(s[i, g_idx[j]]))
            want = O.rne_bf16(np.float32((np.float32(q[i, j]) - z[i, g_idx[j]]) * sc))
            assert w[i, j] == want
    # identity g_idx = the grouped dequantiser
    ident = np.arange(k) // g
    np.testing.assert_array_equal(O.dequantize_weight_act_order(qw, s, z, ident, k),
                                  O.dequantize_weight(qw, s, z, O.WOQ_DTYPE_INT4, k, g))


@pytest.mark.parametrize("act_mode", [O.ACT_PER_TENSOR, O.ACT_PER_M, O.ACT_PER_TENSOR_SYM, O.ACT_PER_M_SYM])
def test_int8_activation_modes_of_the_oracle(act_mode):
    """Codes, scales and zero points of every activation mode reproduce x to half a step, the
    per-tensor modes carry one scale, and the compensated INT8 linear tracks the float one."""
    rng = np.random.default_rng(act_mode)
    x = O.rne_bf16((rng.standard_normal((6, 512)) + 0.4).astype(np.float32))
    q, s, zp = O.dynamic_quant(x, act_mode)
    sym = act_mode in (O.ACT_PER_TENSOR_SYM, O.ACT_PER_M_SYM)
    assert q.dtype == (np.int8 if sym else np.uint8) and (zp is None) == sym
    if act_mode in (O.ACT_PER_TENSOR, O.ACT_PER_TENSOR_SYM):
        assert np.unique(s).size == 1 and (zp is None or np.unique(zp).size == 1)
    back = (q.astype(np.float32) - (0 if zp is None else zp[:, None])) * s[:, None]
    assert np.abs(back - x).max() <= 0.5001 * s.max()
    w = (rng.standard_normal((64, 512)) * 0.02).astype(np.float32)
    qw, sw, _ = O.quantize_per_channel(w, O.WOQ_DTYPE_INT8, sym=True)
    y = O.woq_linear_int8(x, qw, sw, None, act_mode=act_mode)
    ref = x @ (qw.view(np.int8).astype(np.float32) * sw.reshape(-1, 1)).T
    assert np.abs(y - ref).max() <= 0.03 * np.abs(ref).max()


@pytest.mark.parametrize("mode", range(8))
def test_every_activation_quant_mode_against_reference_fake_quant(golden_dir, mode):
    """quantise -> dequantise of the oracle equals the reference test suite's fake-quantiser
    (tests/cpu/test_quantization_default_recipe.py:836-958) for all eight modes, K block 128."""
    f = np.load(os.path.join(golden_dir, "act_quant_modes.npz"))
    for c in range(3):
        x = O.from_bf16_bits(f[f"c{c}.x_bf16"])
        q, sa, zp = O.dynamic_quant_blocks(x, mode, 128)
        K = x.shape[1]
        s_full = np.repeat(sa, 128, axis=1)[:, :K]
        if zp is None:
            dq = q.astype(np.float32) * s_full
        else:
            dq = ((q.astype(np.float32) - np.repeat(zp, 128, axis=1)[:, :K].astype(np.float32)) * s_full).astype(np.float32)
        ref = f[f"c{c}.mode{mode}_f32"]
        if mode in (0, 4):
            # the fixture for the per-tensor modes comes from torch's MinMaxObserver, whose scale
            # rule differs in the last bits ((max - min) / 255 with min, max clamped to include
            # zero); the codes may differ by one step on a few elements
            assert np.abs(dq - ref).max() <= 1.01 * sa.max()
        elif mode >= 5:
            np.testing.assert_array_equal(dq, ref)  # by value: the helper keeps the sign of a zero code
        else:
            # asymmetric: the kernel rounds x / scale + zero_point (one fp32 sum, then
            # nearbyint, woq_dynamic_quant.h:1631-1638) where the test helper rounds x / scale and
            # adds the zero point afterwards; the fp32 sum lands exactly on a half now and then,
            # and the two roundings then differ by one code.  Everything else is identical.
            diff = np.abs(dq - ref)
            assert (diff > 0).mean() <= 0.01
            assert diff.max() <= 1.01 * sa.max()


def test_rmsnorm_restatement_against_torch():
    """oracle.rmsnorm_bf16 (what stands in front of the fused norm + quantiser) against torch's own
    rms_norm in fp32 rounded to bf16: identical except where the fp32 mean differs by summation
    order, and then by one bf16 step."""
    import torch

    rng = np.random.default_rng(5)
    x = O.rne_bf16((rng.standard_normal((33, 1024)) * 2.5 + 0.3).astype(np.float32))
    gamma = O.rne_bf16((rng.random(1024) + 0.5).astype(np.float32))
    got = O.rmsnorm_bf16(x, gamma, 1e-5)
    want = torch.nn.functional.rms_norm(torch.from_numpy(x), (1024,), torch.from_numpy(gamma), 1e-5).bfloat16().float().numpy()
    differ = got != want
    assert differ.mean() < 2e-3, differ.mean()
    np.testing.assert_allclose(got, want, rtol=2.0 ** -7, atol=0)
