"""CPU oracle for the weight-only-quantisation (WOQ) linear path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the arithmetic of the
reference's CPU WOQ linear (intel/intel-extension-for-pytorch).  It is the checker the
parity tests, the smoke test and the CPU-baseline leg of the benchmark compare against;
nothing in the shipped package imports it, and it never stands in for the CUDA path.

Parity status: PINNED.  The functions below are checked against
  * outputs of the reference's own pure-PyTorch quantiser / dequantiser
    (intel_extension_for_pytorch/quantization/_quantize_utils.py:864-1290), executed from
    the reference tree by tests/golden/make_golden.py and stored in tests/golden/*.npz;
  * the reference's AWQ known-answer tensors (tests/cpu/data/awq/*.pt) dequantised with
    the reference test's own dequantize_awq (tests/cpu/test_ipex_llm_quantization.py:35-110);
  * the reference test's activation fake-quantiser
    (tests/cpu/test_quantization_default_recipe.py:915-979).

All file:line citations are paths inside the reference project.

Conventions: N = out features, K = in features, M = tokens, G = group size along K
(G <= 0 means one group per output channel).  bf16 values are carried as float32 arrays
whose low 16 mantissa bits are zero; `to_bf16_bits` gives the uint16 pattern.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

# ---------------------------------------------------------------------------------------
# Constants kept identical to the reference (csrc/cpu/aten/utils/woq_defines.h:6-50,
# intel_extension_for_pytorch/quantization/_qconfig.py:105-165)
# ---------------------------------------------------------------------------------------
WOQ_DTYPE_INT8, WOQ_DTYPE_INT4, WOQ_DTYPE_NF4, WOQ_DTYPE_FP8 = 1, 2, 3, 4
LOWP_MODE_NONE, LOWP_MODE_FP16, LOWP_MODE_BF16, LOWP_MODE_INT8 = 0, 1, 2, 3
QUANT_A_PER_M, QUANT_A_PER_M_SYM = 2, 6
FUSE_NONE, FUSE_GELU_ERF, FUSE_GELU_TANH, FUSE_RELU, FUSE_SILU = 0x0, 0x1, 0x2, 0x3, 0x4
FUSE_ADD, FUSE_ADD_ADD, FUSE_MUL = 0x10, 0x20, 0x30
# Not a reference constant: the fused gate/up epilogue y = silu(gate) * up that the
# reference builds from two ops (transformers/models/cpu/fusions/linear_fusion.py:482-490).
FUSE_SILU_MUL = 0x100

F32_EPS = np.float32(np.finfo(np.float32).eps)


# ---------------------------------------------------------------------------------------
# Rounding helpers
# ---------------------------------------------------------------------------------------
def rne_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even); result stays float32.

    Same rounding as `_mm512_cvtneps_pbh`, which the reference's bf16 tile dequant uses
    (csrc/cpu/tpp/woq/vec.h:301-325), and as ATen's `.to(bfloat16)`.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    nan = np.isnan(x)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = (u + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    out = r.view(np.float32).copy()
    out[nan] = np.nan
    return out


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """uint16 bit pattern of a float32 array that already holds bf16-representable values."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> np.uint32(16)).astype(
        np.uint16
    )


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b).astype(np.uint32) << np.uint32(16)).view(np.float32)


def _round_half_even(x: np.ndarray) -> np.ndarray:
    # torch.round and std::nearbyint (default mode) both round half to even; so does np.rint.
    return np.rint(x)


# ---------------------------------------------------------------------------------------
# a1. Weight quantiser (the input generator of every parity case)
# ---------------------------------------------------------------------------------------
def _qparams(mins, maxs, dtype: int, sym: bool):
    """Scale / zero-point rule shared by per-channel and per-block quantisation
    (quantization/_quantize_utils.py:898-923 and :1054-1076)."""
    zps = None
    if dtype == WOQ_DTYPE_INT8:
        if sym:
            scales = np.maximum(np.abs(maxs), np.abs(mins)) / np.float32(127)
            scales = np.maximum(scales, F32_EPS)
        else:
            scales = (maxs - mins) / np.float32(255)
            scales = np.maximum(scales, F32_EPS)
            zps = -_round_half_even(mins / scales)
            zps = zps - np.float32(128)
    elif dtype == WOQ_DTYPE_INT4:
        if sym:
            scales = np.maximum(np.abs(maxs), np.abs(mins)) / np.float32(7)
            scales = np.maximum(scales, F32_EPS)
        else:
            scales = (maxs - mins) / np.float32(15)
            scales = np.maximum(scales, F32_EPS)
            zps = -_round_half_even(mins / scales)
    elif dtype == WOQ_DTYPE_NF4:
        if not sym:
            raise ValueError("NF4 must be symmetric quant")
        scales = np.maximum(np.maximum(np.abs(maxs), np.abs(mins)), F32_EPS)
    else:
        raise NotImplementedError("FP8 weights come from checkpoints: no quantiser")
    return scales.astype(np.float32), (None if zps is None else zps.astype(np.float32))


# NF4 thresholds and values (quantization/_quantize_utils.py:789-826, woq_utils.h:15-51)
NF4_QUANT_TABLE = np.array([
    -1.0 - 1e-2, -0.8480964004993439, -0.6106329262256622, -0.4599952697753906,
    -0.33967943489551544, -0.23460740596055984, -0.13791173323988914, -0.045525018125772476,
    0.03979014977812767, 0.1202552504837513, 0.2035212516784668, 0.2920137718319893,
    0.3893125355243683, 0.5016634166240692, 0.6427869200706482, 0.8614784181118011], dtype=np.float32)
NF4_DEQUANT_TABLE = np.array([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0], dtype=np.float32)


def map_float_to_nf4(t: np.ndarray) -> np.ndarray:
    """out[t > NF4_QUANT_TABLE[i]] = i for ascending i (quantization/_quantize_utils.py:831-837)."""
    out = np.zeros(t.shape, dtype=np.uint8)
    for i, thr in enumerate(NF4_QUANT_TABLE):
        out[t > thr] = i
    return out


def fp8_e4m3_to_f32(codes: np.ndarray) -> np.ndarray:
    """The reference's byte -> fp32 conversion for FP8 weights (csrc/cpu/aten/utils/woq.h:465-483):
    exponent rebias by 120, three mantissa bits, zero when the low seven bits are zero; no
    special case for NaN or subnormal codes."""
    x = np.ascontiguousarray(codes).view(np.uint8).astype(np.uint32)
    bits = ((x & 7) << 20) | ((((x >> 3) & 15) + 120) << 23)
    bits = np.where((x & 127) == 0, 0, bits) | ((x & 128) << 24)
    return bits.astype(np.uint32).view(np.float32)


def pack_nibbles(q: np.ndarray) -> np.ndarray:
    """[N,K] values 0..15 -> [N,ceil(K/2)] bytes, even k in the low nibble
    (quantization/_quantize_utils.py:1181-1184)."""
    q = q.astype(np.uint8)
    if q.shape[1] % 2:
        q = np.pad(q, ((0, 0), (0, 1)))
    return ((q[:, 1::2] << 4) | (q[:, ::2] & 0xF)).astype(np.uint8)


def unpack_nibbles(qw: np.ndarray) -> np.ndarray:
    """Inverse of pack_nibbles (csrc/cpu/aten/utils/woq_utils.h:94-99)."""
    qw = np.ascontiguousarray(qw).view(np.uint8)
    out = np.empty((qw.shape[0], qw.shape[1] * 2), dtype=np.uint8)
    out[:, ::2] = qw & 0xF
    out[:, 1::2] = qw >> 4
    return out


def quantize_per_block(
    w: np.ndarray, dtype: int, group_size: int, sym: bool = False
) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """Group-wise quantiser (quantization/_quantize_utils.py:1013-1185).

    Returns (qweight, scales[N, ceil(K/G)] f32, zero points[N, ceil(K/G)] f32 or None).
    qweight is [N, ceil(K/2)] uint8 (INT4, nibble-packed) or [N, K] int8.  min/max always
    include zero; values are scaled by the reciprocal of the scale, rounded half-to-even,
    shifted by the zero point (8 for symmetric INT4) and clamped.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    G = group_size
    assert G > 0
    ngroups = (K + G - 1) // G
    scales = np.empty((N, ngroups), dtype=np.float32)
    zps = None if sym else np.empty((N, ngroups), dtype=np.float32)
    q = np.empty((N, K), dtype=np.float32)
    for g in range(ngroups):
        blk = w[:, g * G : min(K, (g + 1) * G)]
        mins = np.minimum(blk.min(axis=1), np.float32(0))
        maxs = np.maximum(blk.max(axis=1), np.float32(0))
        s, z = _qparams(mins, maxs, dtype, sym)
        scales[:, g] = s
        inv = (np.float32(1) / s)[:, None]
        if dtype == WOQ_DTYPE_NF4:
            q[:, g * G : min(K, (g + 1) * G)] = map_float_to_nf4((blk * inv).astype(np.float32))
            continue
        r = _round_half_even(blk * inv)
        if dtype == WOQ_DTYPE_INT8:
            r = r + (z[:, None] if z is not None else np.float32(0))
            r = np.clip(r, -128, 127)
        else:
            r = r + (z[:, None] if z is not None else np.float32(8))
            r = np.clip(r, 0, 15)
        if z is not None:
            zps[:, g] = z
        q[:, g * G : min(K, (g + 1) * G)] = r
    if dtype in (WOQ_DTYPE_INT4, WOQ_DTYPE_NF4):
        return pack_nibbles(q.astype(np.uint8)), scales, zps
    return q.astype(np.int8), scales, zps


def quantize_per_channel(
    w: np.ndarray, dtype: int, sym: bool = False
) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """Per-output-channel quantiser (quantization/_quantize_utils.py:864-946).
    Scales / zero points have shape [N]."""
    qw, s, z = quantize_per_block(w, dtype, w.shape[1], sym)
    return qw, s[:, 0].copy(), (None if z is None else z[:, 0].copy())


# ---------------------------------------------------------------------------------------
# Low-precision-checkpoint layouts (GPTQ / AWQ int32 packing)
# ---------------------------------------------------------------------------------------
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def awq_unpack_int32(packed: np.ndarray) -> np.ndarray:
    """AWQ int32 packing: [R, C/8] int32 -> [R, C] values 0..15.  Nibble j of a word
    holds logical column 8*c + AWQ_ORDER[j] (csrc/cpu/aten/kernels/WoqUtilKrnl.cpp:140-217;
    tests/cpu/test_ipex_llm_quantization.py:8-32)."""
    p = np.ascontiguousarray(packed).view(np.uint32)
    R, C8 = p.shape
    out = np.empty((R, C8, 8), dtype=np.uint8)
    for j in range(8):
        out[:, :, AWQ_ORDER[j]] = ((p >> np.uint32(4 * j)) & np.uint32(0xF)).astype(np.uint8)
    return out.reshape(R, C8 * 8)


def awq_to_plain(
    qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """AWQ checkpoint (qweight [K,N/8] i32, qzeros [K/G,N/8] i32, scales [K/G,N]) ->
    plain (nibble-packed [N,K/2] u8, scales [N,K/G], zero points [N,K/G] f32)."""
    q_kn = awq_unpack_int32(qweight)  # [K, N]
    z_gn = awq_unpack_int32(qzeros)  # [K/G, N]
    return (
        pack_nibbles(np.ascontiguousarray(q_kn.T)),
        np.ascontiguousarray(np.asarray(scales).T),
        np.ascontiguousarray(z_gn.T).astype(np.float32),
    )


def gptq_unpack_int32_rows(packed: np.ndarray) -> np.ndarray:
    """GPTQ int32 packing along rows: [R/8, C] int32 -> [R, C]; nibble j of word r holds
    row 8*r + j (csrc/cpu/aten/kernels/WoqUtilKrnl.cpp:109-139)."""
    p = np.ascontiguousarray(packed).view(np.uint32)
    R8, C = p.shape
    out = np.empty((R8, 8, C), dtype=np.uint8)
    for j in range(8):
        out[:, j, :] = ((p >> np.uint32(4 * j)) & np.uint32(0xF)).astype(np.uint8)
    return out.reshape(R8 * 8, C)


# ---------------------------------------------------------------------------------------
# Dequantisation (a3 + a7 + a11)
# ---------------------------------------------------------------------------------------
def _expand_groups(v: np.ndarray, K: int, G: int) -> np.ndarray:
    v = np.asarray(v, dtype=np.float32)
    if v.ndim == 1:
        v = v[:, None]
    if v.shape[1] == 1:
        return np.broadcast_to(v, (v.shape[0], K))
    return np.repeat(v, G, axis=1)[:, :K]


def weight_integers(qweight: np.ndarray, dtype: int, K: int) -> np.ndarray:
    """Stored integer code of every weight as float32 [N,K] (0..15 or -128..127)."""
    if dtype == WOQ_DTYPE_INT4:
        return unpack_nibbles(qweight)[:, :K].astype(np.float32)
    if dtype == WOQ_DTYPE_INT8:
        return np.ascontiguousarray(qweight).view(np.int8)[:, :K].astype(np.float32)
    if dtype == WOQ_DTYPE_NF4:
        return NF4_DEQUANT_TABLE[unpack_nibbles(qweight)[:, :K]]
    if dtype == WOQ_DTYPE_FP8:
        return fp8_e4m3_to_f32(qweight)[:, :K]
    raise NotImplementedError


def dequantize_weight(
    qweight: np.ndarray,
    scales: np.ndarray,
    zps: Optional[np.ndarray],
    dtype: int,
    K: int,
    group_size: int,
    scale_rounding: str = "bf16",
    round_output: bool = True,
) -> np.ndarray:
    """Dequantised weight [N,K] (float32 array holding bf16 values when round_output).

    W = RNE_bf16((q - zp) * scale'), computed in fp32 with one multiply and one rounding,
    where scale' depends on `scale_rounding`:
      "bf16": scale' = RNE_bf16(float(scale)) -- the bf16 tile dequant
              (csrc/cpu/aten/utils/woq.h:1223-1325,1501-1581 with the bf16 scale copy made at
              csrc/cpu/jit/cpu/kernels/ContextLinearWoq.h:60-115) and the cached large-batch
              weight (csrc/cpu/jit/cpu/kernels/LinearWoqPacked.cpp:456-477);
      "none": scale' = float(scale) -- the plain ATen kernel
              (csrc/cpu/aten/utils/woq.h:3564-3566, woq_utils.h:79-163);
      "fp16": scale' = float(fp16(scale)) -- the small-M fp16 kernel (woq.h:784-951).
    A missing zero point means symmetric storage: 8 for INT4, 0 for INT8
    (woq_utils.h:110-112, 121-123).
    """
    G = K if group_size <= 0 else group_size
    q = weight_integers(qweight, dtype, K)
    s = np.asarray(scales, dtype=np.float32)
    if scale_rounding == "bf16":
        s = rne_bf16(s)
    elif scale_rounding == "fp16":
        s = s.astype(np.float16).astype(np.float32)
    elif scale_rounding != "none":
        raise ValueError(scale_rounding)
    s_full = _expand_groups(s, K, G)
    if zps is None:
        z_full = np.float32(8.0 if dtype == WOQ_DTYPE_INT4 else 0.0)
    else:
        z_full = _expand_groups(zps, K, G)
    w = (q - z_full) * s_full
    w = w.astype(np.float32)
    return rne_bf16(w) if round_output else w


def _round_to(v: np.ndarray, compute: str) -> np.ndarray:
    v = np.asarray(v, dtype=np.float32)
    if compute == "bf16":
        return rne_bf16(v)
    if compute == "fp16":
        return v.astype(np.float16).astype(np.float32)
    if compute == "fp32":
        return v
    raise ValueError(compute)


def woq_linear_any(x, qweight, scales, zps, bias, dtype: int, group_size: int, compute: str, io: str,
                   fusion: int = FUSE_NONE, others: Sequence[np.ndarray] = ()) -> np.ndarray:
    """The floating-point routes of qlinear_woq_affine for every weight dtype
    (csrc/cpu/aten/kernels/WoqLinearKrnl.cpp:75-165): compute in `compute` ("bf16", "fp16" or
    "fp32"), activations / outputs / extra tensors of dtype `io`.

    W = round((code - zp) * round(scale)), x rounded to the compute dtype, fp32 accumulation over
    the whole K, + bias, rounded to `io`, post-op on `io` data (one rounding per operation).
    For compute == io == "bf16" and INT4 / INT8 weights this is woq_linear_bf16."""
    K = x.shape[1]
    G = K if group_size <= 0 else group_size
    q = weight_integers(qweight, dtype, K)
    s_full = _expand_groups(_round_to(scales, compute), K, G)
    if zps is None:
        z_full = np.float32(8.0 if dtype == WOQ_DTYPE_INT4 else 0.0)
    else:
        z_full = _expand_groups(zps, K, G)
    w = _round_to(((q - z_full) * s_full).astype(np.float32), compute)
    acc = _round_to(x, compute) @ w.T
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=np.float32)[None, :]
    y = _round_to(acc, io)
    r = lambda v: _round_to(v, io)  # noqa: E731
    if fusion == FUSE_NONE:
        return y
    if fusion == FUSE_GELU_ERF:
        y64 = y.astype(np.float64)
        return r((0.5 * y64 * (1.0 + _erf(y64 / math.sqrt(2.0)))).astype(np.float32))
    if fusion == FUSE_GELU_TANH:
        y64 = y.astype(np.float64)
        return r((0.5 * y64 * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (y64 + 0.044715 * y64**3)))).astype(np.float32))
    if fusion == FUSE_RELU:
        return np.maximum(y, np.float32(0))
    if fusion == FUSE_SILU:
        sig = r((1.0 / (1.0 + np.exp(-y.astype(np.float64)))).astype(np.float32))
        return r(y * sig)
    if fusion in (FUSE_ADD, FUSE_ADD_ADD):
        for t in others[: 1 if fusion == FUSE_ADD else 2]:
            y = r(y + np.asarray(t, dtype=np.float32).reshape(y.shape))
        return y
    if fusion == FUSE_MUL:
        return r(y * np.asarray(others[0], dtype=np.float32).reshape(y.shape))
    raise ValueError(f"unexpected fusion type {fusion:#x}")


# ---------------------------------------------------------------------------------------
# a10. Post-ops, applied to the bf16 result (csrc/cpu/aten/utils/woq.h:2924-2945)
# ---------------------------------------------------------------------------------------
_erf = np.vectorize(math.erf, otypes=[np.float64])


def _silu_bf16(y: np.ndarray) -> np.ndarray:
    # sigmoid is rounded to bf16 before the product, the product is rounded again
    # (csrc/cpu/tpp/xsmm_functors.h:2620-2657: SiLUFwdTPP = sigmoid TPP then mul TPP, both
    # with bf16 outputs and fp32 internal arithmetic).
    y64 = y.astype(np.float64)
    sig = rne_bf16((1.0 / (1.0 + np.exp(-y64))).astype(np.float32))
    return rne_bf16(y * sig)


def dequantize_weight_act_order(qweight, scales, zps, g_idx, K: int) -> np.ndarray:
    """GPTQ act-order: input channel k belongs to group g_idx[k], so
    W[n][k] = RNE_bf16((q[n][k] - zp[n][g_idx[k]]) * RNE_bf16(scale[n][g_idx[k]])).
    The reference reaches the same values by shuffling the weight's input channels so that
    every group is contiguous and shuffling the activations alike
    (csrc/cpu/jit/cpu/kernels/LinearWoqPacked.cpp:755-870, 405-420)."""
    g = np.asarray(g_idx).astype(np.int64)
    q = weight_integers(qweight, WOQ_DTYPE_INT4, K)
    s = rne_bf16(np.asarray(scales, dtype=np.float32))[:, g]
    z = np.float32(8.0) if zps is None else np.asarray(zps, dtype=np.float32)[:, g]
    return rne_bf16(((q - z) * s).astype(np.float32))


def woq_linear_bf16_act_order(x, qweight, scales, zps, bias, g_idx):
    """y = bf16(x W^T + bias) with the act-order weight above, fp32 accumulation."""
    x = np.asarray(x, dtype=np.float32)
    w = dequantize_weight_act_order(qweight, scales, zps, g_idx, x.shape[1])
    y = x.astype(np.float64) @ w.astype(np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[None, :]
    return rne_bf16(y.astype(np.float32))


def apply_post_op(y: np.ndarray, fusion: int, others: Sequence[np.ndarray] = ()) -> np.ndarray:
    """y is a float32 array of bf16 values [M,N]; returns the same kind of array."""
    if fusion == FUSE_NONE:
        return y
    if fusion == FUSE_GELU_ERF:
        # The reference's TPP uses a minimax erf approximation whose coefficients live in
        # libxsmm (not in the reference tree); the exact erf form is what its tests compare
        # against (tests/cpu/test_quantization_default_recipe.py:612-677).
        y64 = y.astype(np.float64)
        return rne_bf16((0.5 * y64 * (1.0 + _erf(y64 / math.sqrt(2.0)))).astype(np.float32))
    if fusion == FUSE_GELU_TANH:
        y64 = y.astype(np.float64)
        inner = math.sqrt(2.0 / math.pi) * (y64 + 0.044715 * y64**3)
        return rne_bf16((0.5 * y64 * (1.0 + np.tanh(inner))).astype(np.float32))
    if fusion == FUSE_RELU:
        return np.maximum(y, np.float32(0))
    if fusion == FUSE_SILU:
        return _silu_bf16(y)
    if fusion in (FUSE_ADD, FUSE_ADD_ADD):
        n = 1 if fusion == FUSE_ADD else 2
        for t in others[:n]:
            y = rne_bf16(y + np.asarray(t, dtype=np.float32).reshape(y.shape))
        return y
    if fusion == FUSE_MUL:
        return rne_bf16(y * np.asarray(others[0], dtype=np.float32).reshape(y.shape))
    raise ValueError(f"unexpected fusion type {fusion:#x}")


# ---------------------------------------------------------------------------------------
# a7 / a11. bf16-compute WOQ linear (WoqLowpMode.BF16)
# ---------------------------------------------------------------------------------------
def woq_linear_bf16(
    x: np.ndarray,
    qweight: np.ndarray,
    scales: np.ndarray,
    zps: Optional[np.ndarray],
    bias: Optional[np.ndarray],
    dtype: int,
    group_size: int,
    fusion: int = FUSE_NONE,
    others: Sequence[np.ndarray] = (),
    scale_rounding: str = "bf16",
    return_f32: bool = False,
) -> np.ndarray:
    """y[M,N] for bf16 activations x[M,K] (float32 array of bf16 values).

    y = bf16( sum_k x[m,k] * Wdq[n,k]  (+ bias[n]) ), fp32 accumulation over the whole K
    (csrc/cpu/aten/utils/woq.h:1801-1964 feeding a bf16->fp32 BRGEMM; bias preloaded in fp32
    at :3285-3311; final fp32->bf16 conversion at :3450-3462), then the post-op on the bf16
    value.  With FUSE_SILU_MUL the weight holds gate rows [0,N/2) and up rows [N/2,N) and
    the result is bf16(up * silu(gate)) [M,N/2], which is what the two-op composition
    woq_linear_silu + woq_linear_mul produces (linear_fusion.py:482-490).
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    w = dequantize_weight(qweight, scales, zps, dtype, K, group_size, scale_rounding)
    return linear_from_dequantised(x, w, bias, fusion, others, return_f32)


def linear_from_dequantised(x, w, bias=None, fusion: int = FUSE_NONE, others: Sequence[np.ndarray] = (),
                            return_f32: bool = False) -> np.ndarray:
    """The second half of woq_linear_bf16 for a weight that is already dequantised (a caller
    that applies one large layer to several inputs dequantises it once)."""
    acc = np.ascontiguousarray(x, dtype=np.float32) @ w.T  # fp32 accumulate
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=np.float32)[None, :]
    if return_f32:
        return acc.astype(np.float32)
    y = rne_bf16(acc)
    if fusion == FUSE_SILU_MUL:
        half = y.shape[1] // 2
        return rne_bf16(y[:, half:] * _silu_bf16(y[:, :half]))
    return apply_post_op(y, fusion, others)


def rmsnorm_bf16(x: np.ndarray, gamma: np.ndarray, eps: float) -> np.ndarray:
    """y = bf16(x * rsqrt(mean(x^2) + eps) * gamma), fp32 arithmetic and one rounding: what stands in
    front of the q/k/v and gate/up linears of a Llama-style block (stock torch rms_norm in the
    reference's model rewrites; the reference has no fused norm + quantiser, this restates the
    unfused pair for the B200 side's fusion).  x [M, K] and gamma [K] hold bf16 values."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    ms = (x * x).sum(axis=1, dtype=np.float32) / np.float32(x.shape[1])
    inv = (np.float32(1.0) / np.sqrt(ms + np.float32(eps))).astype(np.float32)
    return rne_bf16((x * inv[:, None]).astype(np.float32) * np.asarray(gamma, dtype=np.float32)[None, :])


# ---------------------------------------------------------------------------------------
# a8. Dynamic per-token activation quantisation (WoqLowpMode.INT8)
# ---------------------------------------------------------------------------------------
def dynamic_quant_per_token(
    x: np.ndarray, sym: bool = True
) -> Tuple[np.ndarray, np.ndarray, Optional[np.ndarray]]:
    """Per-row quantisation of bf16 activations to int8 (sym) / uint8 (asym)
    (csrc/cpu/aten/utils/woq_dynamic_quant.h:1526-1750, modes QUANT_A_PER_M[_SYM]).

    sym : scale = max(|max|,|min|)/127 ; q = clamp(nearbyint(x/scale), -128, 127)
    asym: scale = (max-min)/255 ; zp = -nearbyint(min/scale) ; q = clamp(nearbyint(x/scale + zp), 0, 255)
    True division, round-half-even, no zero clamp of min/max and no epsilon.  A row of all
    zeros gives scale 0; the reference then divides by zero -- the oracle (and the CUDA
    kernel) define that row's codes as 0.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    mn = x.min(axis=1)
    mx = x.max(axis=1)
    if sym:
        scale = (np.maximum(np.abs(mx), np.abs(mn)) / np.float32(127)).astype(np.float32)
        zp = None
        safe = np.where(scale > 0, scale, np.float32(1))
        q = _round_half_even((x / safe[:, None]).astype(np.float32))
        q = np.clip(q, -128, 127)
        q[scale == 0] = 0
        return q.astype(np.int8), scale, None
    scale = ((mx - mn) / np.float32(255)).astype(np.float32)
    safe = np.where(scale > 0, scale, np.float32(1))
    zp = (-_round_half_even((mn / safe).astype(np.float32))).astype(np.int32)
    q = _round_half_even(((x / safe[:, None]).astype(np.float32) + zp[:, None].astype(np.float32)))
    q = np.clip(q, 0, 255)
    q[scale == 0] = 0
    return q.astype(np.uint8), scale, zp


ACT_PER_TENSOR, ACT_PER_M, ACT_PER_TENSOR_SYM, ACT_PER_M_SYM = 0, 2, 4, 6  # woq_defines.h:11-19


def dynamic_quant(x: np.ndarray, act_mode: int = ACT_PER_M_SYM):
    """Activation codes, scales [M] and zero points [M] (None when symmetric) for the
    per-token modes (2, 6) and the per-tensor modes (0, 4): the per-tensor ones take one range
    over the whole activation tensor and every row carries the same scale and zero point."""
    sym = act_mode in (ACT_PER_TENSOR_SYM, ACT_PER_M_SYM)
    if act_mode in (ACT_PER_M, ACT_PER_M_SYM):
        return dynamic_quant_per_token(x, sym=sym)
    assert act_mode in (ACT_PER_TENSOR, ACT_PER_TENSOR_SYM), act_mode
    x = np.ascontiguousarray(x, dtype=np.float32)
    q, scale, zp = dynamic_quant_per_token(x.reshape(1, -1), sym=sym)
    m = x.shape[0]
    return q.reshape(x.shape), np.repeat(scale, m), None if zp is None else np.repeat(zp, m)


# ---------------------------------------------------------------------------------------
# a9. INT8 x INT8 -> INT32 WOQ linear (WoqLowpMode.INT8, INT8 symmetric per-channel weights)
# ---------------------------------------------------------------------------------------
INT8_BLOCK_K = 128  # get_block_k for lowp INT8 (csrc/cpu/aten/Linear.cpp:362-376)


def int8_accumulators(qa: np.ndarray, qw: np.ndarray) -> np.ndarray:
    """Exact int32 accumulators acc[m,n] = sum_k qa[m,k]*qw[n,k] over the whole K.
    Computed with a float64 matrix product, which is exact here (|sum| < 2^53)."""
    a = qa.astype(np.float64)
    w = np.ascontiguousarray(qw).view(np.int8).astype(np.float64)
    return np.rint(a @ w.T).astype(np.int64).astype(np.int32)


def woq_linear_int8(
    x: np.ndarray,
    qweight: np.ndarray,
    scales: np.ndarray,
    bias: Optional[np.ndarray],
    fusion: int = FUSE_NONE,
    others: Sequence[np.ndarray] = (),
    block_k: int = INT8_BLOCK_K,
    return_acc: bool = False,
    act_mode: int = ACT_PER_M_SYM,
):
    """INT8 weights (symmetric, per channel), dynamically quantised activations (per token or
    per tensor, symmetric or asymmetric).

    Per K block of 128: qC = sum_k qa*qw (int32, exact); C += (float(qC - comp[n] * zp_a[m]) *
    scale_a[m]) * scale_w[n] in fp32 with comp[n] the block's sum of weight codes (the term
    is absent for symmetric activations), blocks taken in k order after the fp32 bias
    (csrc/cpu/aten/utils/woq.h:2231-2354; driver loop :3312-3448), then fp32 -> bf16 and the
    post-op.  With return_acc also the whole-K accumulators before compensation, the codes,
    scales and zero points.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    qw = np.ascontiguousarray(qweight).view(np.int8)
    N = qw.shape[0]
    qa, sa, zpa = dynamic_quant(x, act_mode)
    sw = np.asarray(scales, dtype=np.float32).reshape(N)
    C = np.zeros((M, N), dtype=np.float32)
    if bias is not None:
        C += np.asarray(bias, dtype=np.float32)[None, :]
    qa64 = qa.astype(np.float64)  # float64 products and sums of int8 codes are exact
    qw64 = qw.astype(np.float64)
    for k0 in range(0, K, block_k):
        qc = qa64[:, k0 : k0 + block_k] @ qw64[:, k0 : k0 + block_k].T
        if zpa is not None:
            comp = qw64[:, k0 : k0 + block_k].sum(axis=1)
            qc = qc - zpa.astype(np.float64)[:, None] * comp[None, :]
        qc = qc.astype(np.float32)
        C = (C + ((qc * sa[:, None]).astype(np.float32) * sw[None, :]).astype(np.float32)).astype(
            np.float32
        )
    y = rne_bf16(C)
    if fusion == FUSE_SILU_MUL:
        half = y.shape[1] // 2
        y = rne_bf16(y[:, half:] * _silu_bf16(y[:, :half]))
    else:
        y = apply_post_op(y, fusion, others)
    if return_acc:
        if zpa is not None:
            return y, int8_accumulators(qa, qw), qa, sa, zpa
        return y, int8_accumulators(qa, qw), qa, sa
    return y


# ---------------------------------------------------------------------------------------
# a8 / a9 in general: every activation quantisation mode, INT4 or INT8 weights, K blocks
# ---------------------------------------------------------------------------------------
def int8_block_k(K: int, group_size: int) -> int:
    """get_block_k for lowp INT8: min(group, 128), halved until it divides K
    (csrc/cpu/aten/Linear.cpp:362-376)."""
    kb = min(group_size, 128) if group_size > 0 else 128
    while K % kb:
        kb //= 2
    return kb


def dynamic_quant_blocks(x: np.ndarray, act_mode: int, block_k: int):
    """Activation codes [M, K] and, per token and K block, scales [M, Kc] and zero points
    [M, Kc] (None when symmetric) for all eight modes of the reference
    (csrc/cpu/aten/utils/woq_defines.h:11-19, woq_dynamic_quant.h:1526-1750):
      0 / 4  one range for the whole tensor          1 / 5  one per K block, shared by all tokens
      2 / 6  one per token                            3 / 7  one per token and K block
    (+4: symmetric int8 codes; else uint8 codes with a zero point).  Every mode is the per-token
    rule of dynamic_quant_per_token applied to the elements that share a range."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    Kc = (K + block_k - 1) // block_k
    sym = act_mode >= 4
    base = act_mode & 3
    q = np.empty((M, K), dtype=np.int8 if sym else np.uint8)
    sa = np.empty((M, Kc), dtype=np.float32)
    zp = None if sym else np.empty((M, Kc), dtype=np.int32)
    if base in (0, 2):
        qq, s, z = dynamic_quant(x, act_mode)
        q[:] = qq
        sa[:] = s[:, None]
        if zp is not None:
            zp[:] = z[:, None]
        return q, sa, zp
    for c in range(Kc):
        blk = x[:, c * block_k : (c + 1) * block_k]
        if base == 1:   # all tokens share the block's range
            qq, s, z = dynamic_quant_per_token(blk.reshape(1, -1), sym=sym)
            q[:, c * block_k : (c + 1) * block_k] = qq.reshape(blk.shape)
            sa[:, c] = s[0]
            if zp is not None:
                zp[:, c] = z[0]
        else:
            qq, s, z = dynamic_quant_per_token(blk, sym=sym)
            q[:, c * block_k : (c + 1) * block_k] = qq
            sa[:, c] = s
            if zp is not None:
                zp[:, c] = z
    return q, sa, zp


def woq_linear_int8_blocks(x, qweight, wdtype: int, scales, zps_w, bias, group_size: int, act_mode: int,
                           fusion: int = FUSE_NONE, others: Sequence[np.ndarray] = (), return_blocks: bool = False):
    """WoqLowpMode.INT8 for INT4 or INT8 weights with per-channel or per-group scales and any
    activation quantisation mode.  Per K block (int8_block_k):
        qC[m,n] = sum_k qa[m,k] * (qw[n,k] - zp_w[n,g])                      int32, exact
        qC     -= comp[n] * zp_a[m,block],  comp[n] = sum_k (qw[n,k] - zp_w[n,g])   (asymmetric activations)
        C[m,n] += (float(qC) * scale_a[m,block]) * scale_w[n,g]              fp32, blocks in k order
    after the fp32 bias; then fp32 -> bf16 and the post-op
    (csrc/cpu/aten/utils/woq.h:962-1126 for 4-bit weights, :2231-2354 for INT8 weights).
    With return_blocks also the int32 block accumulators [Kc, M, N] (after the compensation)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    M, K = x.shape
    G = K if group_size <= 0 else group_size
    kb = int8_block_k(K, group_size)
    qw = weight_integers(qweight, wdtype, K).astype(np.float64)
    N = qw.shape[0]
    if zps_w is None:
        zw = np.full((N, (K + G - 1) // G), 8.0 if wdtype == WOQ_DTYPE_INT4 else 0.0)
    else:
        zw = np.asarray(zps_w, dtype=np.float64).reshape(N, -1)
    sw = np.asarray(scales, dtype=np.float32).reshape(N, -1)
    qa, sa, zpa = dynamic_quant_blocks(x, act_mode, kb)
    qa64 = qa.astype(np.float64)
    C = np.zeros((M, N), dtype=np.float32)
    if bias is not None:
        C += np.asarray(bias, dtype=np.float32)[None, :]
    blocks = []
    for c, k0 in enumerate(range(0, K, kb)):
        g = k0 // G
        wb = qw[:, k0 : k0 + kb] - zw[:, g][:, None]
        qc = qa64[:, k0 : k0 + kb] @ wb.T
        if zpa is not None:
            qc = qc - zpa[:, c].astype(np.float64)[:, None] * wb.sum(axis=1)[None, :]
        if return_blocks:
            blocks.append(np.rint(qc).astype(np.int64).astype(np.int32))
        qc = qc.astype(np.float32)
        C = (C + ((qc * sa[:, c][:, None]).astype(np.float32) * sw[:, g][None, :]).astype(np.float32)).astype(np.float32)
    y = rne_bf16(C)
    if fusion == FUSE_SILU_MUL:
        half = y.shape[1] // 2
        y = rne_bf16(y[:, half:] * _silu_bf16(y[:, :half]))
    else:
        y = apply_post_op(y, fusion, others)
    if return_blocks:
        return y, np.stack(blocks), qa, sa, zpa
    return y


# ---------------------------------------------------------------------------------------
# a14. Mixtral MoE layer built from WOQ linears
# ---------------------------------------------------------------------------------------
def moe_route_top2(h: np.ndarray, router_w: np.ndarray):
    """softmax(fp32) over bf16 router logits, top-2, renormalise, cast to bf16
    (transformers/models/reference/modules/decoder.py:919-951)."""
    logits = rne_bf16(h @ np.asarray(router_w, dtype=np.float32).T)
    z = logits - logits.max(axis=1, keepdims=True)
    p = np.exp(z.astype(np.float32))
    p = (p / p.sum(axis=1, keepdims=True)).astype(np.float32)
    idx = np.argsort(-p, axis=1, kind="stable")[:, :2]
    top = np.take_along_axis(p, idx, axis=1)
    top = (top / top.sum(axis=1, keepdims=True)).astype(np.float32)
    return idx.astype(np.int32), rne_bf16(top)


def moe_layer(h, topk_idx, topk_w, experts, group_size):
    """out[t] = sum over the token's experts, in expert order, of
    bf16(float(out[t]) + float(y_e[t]) * float(w_bf16))  with
    y_e = w2( bf16(up(x) * silu(gate(x))) )
    (csrc/cpu/aten/kernels/MoEKrnl.cpp:67-120,254-285).
    experts[e] = dict(w13=(q,s,z), w2=(q,s,z)); w13 stacks gate rows then up rows."""
    T = h.shape[0]
    Hd = experts[0]["w2"][0].shape[0]
    out = np.zeros((T, Hd), dtype=np.float32)
    for e, ex in enumerate(experts):
        sel_t, sel_j = np.nonzero(topk_idx == e)
        if sel_t.size == 0:
            continue
        xe = h[sel_t]
        q, s, z = ex["w13"]
        a = woq_linear_bf16(xe, q, s, z, None, WOQ_DTYPE_INT4, group_size, FUSE_SILU_MUL)
        q, s, z = ex["w2"]
        y = woq_linear_bf16(a, q, s, z, None, WOQ_DTYPE_INT4, group_size)
        w = topk_w[sel_t, sel_j][:, None]
        out[sel_t] = rne_bf16(out[sel_t] + y * w)
    return out


# ---------------------------------------------------------------------------------------
# a15. Row-parallel linear followed by all-reduce and bias
# ---------------------------------------------------------------------------------------
def row_parallel_linear(x, qweight_shards, scales_shards, zps_shards, bias, dtype, group_size):
    """Each rank r computes bf16 y_r from its K shard; the ranks' bf16 outputs are summed
    in fp32 and rounded to bf16 once, then the bias is added
    (nn/modules/weight_only_quantization.py:605-633;
    csrc/cpu/aten/kernels/TPPSHMAllreduceAddKrnl.cpp:183-197)."""
    p = len(qweight_shards)
    K = x.shape[1]
    ks = K // p
    acc = None
    for r in range(p):
        y = woq_linear_bf16(
            x[:, r * ks : (r + 1) * ks],
            qweight_shards[r],
            scales_shards[r],
            None if zps_shards is None else zps_shards[r],
            None,
            dtype,
            group_size,
        )
        acc = y if acc is None else acc + y
    y = rne_bf16(acc)
    if bias is not None:
        y = rne_bf16(y + np.asarray(bias, dtype=np.float32)[None, :])
    return y


# ---------------------------------------------------------------------------------------
# Parity metrics
# ---------------------------------------------------------------------------------------
def parity_metrics(y: np.ndarray, y_ref: np.ndarray) -> Tuple[float, float]:
    """(max |y - y_ref| / max |y_ref|,  mean |y - y_ref| / mean |y_ref|)."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    d = np.abs(y - y_ref)
    return float(d.max() / max(np.abs(y_ref).max(), 1e-30)), float(
        d.mean() / max(np.abs(y_ref).mean(), 1e-30)
    )


MAX_ABS_TOL = 1e-2  # max-abs error <= 1e-2 * ||y_ref||_inf
MEAN_REL_TOL = 2e-3  # mean relative error <= 2e-3
