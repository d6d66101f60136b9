"""Weight quantisers of the WOQ path, device-agnostic torch code.

Same rules as the reference's quantize_per_channel / quantize_per_block /
dequantize_per_channel / dequantize_per_block
(intel_extension_for_pytorch/quantization/_quantize_utils.py:864-1290): min/max include zero,
scale = (max - min) / 15 (INT4 asym), max|w| / 7 (INT4 sym), max|w| / 127 (INT8 sym),
(max - min) / 255 (INT8 asym, zero point shifted by -128), clamped below by fp32 eps;
values are multiplied by the reciprocal scale, rounded half to even, shifted by the zero
point (8 for symmetric INT4) and clamped; INT4 codes are packed two per byte, even k low.
NF4 (symmetric only): scale = max|w|, code = the number of the last threshold of the
reference's NF4_QUANT_TABLE below w / scale (:789-846).
Written group-parallel so that it runs at memory speed on a GPU.
"""
from typing import Optional, Tuple

import torch

from ._qconfig import WoqWeightDtype


# thresholds / values of the 16 NF4 codes (reference: quantization/_quantize_utils.py:789-826)
NF4_QUANT_TABLE = [
    -1.0 - 1e-2, -0.8480964004993439, -0.6106329262256622, -0.4599952697753906,
    -0.33967943489551544, -0.23460740596055984, -0.13791173323988914, -0.045525018125772476,
    0.03979014977812767, 0.1202552504837513, 0.2035212516784668, 0.2920137718319893,
    0.3893125355243683, 0.5016634166240692, 0.6427869200706482, 0.8614784181118011,
]
NF4_DEQUANT_TABLE = [
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453,
    -0.28444138169288635, -0.18477343022823334, -0.09105003625154495, 0.0,
    0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
    0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0,
]


def is_4bit(dtype) -> bool:
    return dtype in (WoqWeightDtype.INT4, WoqWeightDtype.NF4)


def _qparams(mins, maxs, dtype, sym_quant):
    eps = torch.finfo(torch.float32).eps
    zps = None
    if dtype == WoqWeightDtype.INT8:
        if sym_quant:
            scales = torch.maximum(maxs.abs(), mins.abs()) / 127
            scales = scales.clamp_min(eps)
        else:
            scales = ((maxs - mins) / 255).clamp_min(eps)
            zps = -torch.round(mins / scales) - 128
    elif dtype == WoqWeightDtype.INT4:
        if sym_quant:
            scales = (torch.maximum(maxs.abs(), mins.abs()) / 7).clamp_min(eps)
        else:
            scales = ((maxs - mins) / 15).clamp_min(eps)
            zps = -torch.round(mins / scales)
    elif dtype == WoqWeightDtype.NF4:
        assert sym_quant, "NF4 must be symmetric quant"
        scales = torch.maximum(maxs.abs(), mins.abs()).clamp_min(eps)
    else:
        raise NotImplementedError("FP8 weights come from checkpoints, there is no FP8 quantiser")
    return scales, zps


def _pack_int4(q: torch.Tensor) -> torch.Tensor:
    if q.size(-1) % 2:
        q = torch.nn.functional.pad(q, (0, 1), value=0)
    return (q[:, 1::2] << 4 | (q[:, ::2] & 0xF)).contiguous()


def _quantize_groups(t, dtype, scales, zps, sym_quant):
    inv = 1 / scales.unsqueeze(-1)
    if dtype == WoqWeightDtype.NF4:
        # the last threshold below the value: thresholds ascend, so count them
        v = t * inv
        table = torch.tensor(NF4_QUANT_TABLE, dtype=torch.float32, device=t.device)
        code = (v.unsqueeze(-1) > table).sum(dim=-1) - 1
        return code.clamp_(0, 15)
    r = torch.round(t * inv)
    if dtype == WoqWeightDtype.INT8:
        if zps is not None:
            r = r + zps.unsqueeze(-1)
        return r.clamp_(-128, 127)
    r = r + (zps.unsqueeze(-1) if zps is not None else 8)
    return r.clamp_(0, 15)


def quantize_per_channel(t: torch.Tensor, dtype, scales=None, zero_points=None, sym_quant=False):
    """[N, K] float -> (qweight, scales [N], zero points [N] or None)."""
    assert t.ndim == 2
    t = t.float()
    if scales is None or (not sym_quant and zero_points is None):
        zero = torch.zeros((), device=t.device)
        mins = torch.minimum(t.amin(dim=1), zero)
        maxs = torch.maximum(t.amax(dim=1), zero)
        scales, zero_points = _qparams(mins, maxs, dtype, sym_quant)
    q = _quantize_groups(t, dtype, scales, None if sym_quant else zero_points, sym_quant)
    if is_4bit(dtype):
        return _pack_int4(q.to(torch.uint8)), scales, zero_points
    return q.to(torch.int8).contiguous(), scales, zero_points


def quantize_per_block(input: torch.Tensor, dtype, group_size, scales=None, zero_points=None,
                       sym_quant=False):
    """[N, K] float -> (qweight, scales [N, ceil(K/G)], zero points [N, ceil(K/G)] or None)."""
    assert input.dim() == 2 and group_size > 0
    t = input.float()
    N, K = t.shape
    G = group_size
    ng = (K + G - 1) // G
    pad = ng * G - K
    if pad:
        # a short last group: pad with its own first value so min / max are unchanged, cut later
        tail = t[:, (ng - 1) * G :]
        t = torch.cat([t, tail[:, :1].expand(N, pad)], dim=1)
    tg = t.view(N, ng, G)
    if scales is None or (not sym_quant and zero_points is None):
        zero = torch.zeros((), device=t.device)
        mins = torch.minimum(tg.amin(dim=-1), zero)
        maxs = torch.maximum(tg.amax(dim=-1), zero)
        scales, zero_points = _qparams(mins, maxs, dtype, sym_quant)
    q = _quantize_groups(tg, dtype, scales, None if sym_quant else zero_points, sym_quant)
    q = q.view(N, ng * G)[:, :K]
    if is_4bit(dtype):
        return _pack_int4(q.to(torch.uint8)), scales, zero_points
    return q.to(torch.int8).contiguous(), scales, zero_points


def _unpack_int4(qt: torch.Tensor) -> torch.Tensor:
    out = torch.empty(qt.shape[0], qt.shape[1] * 2, dtype=torch.uint8, device=qt.device)
    out[:, ::2] = qt & 0xF
    out[:, 1::2] = qt >> 4
    return out


def dequantize_per_channel(qt, scales, zps: Optional[torch.Tensor], dtype, weight_shape=None):
    scales = scales.reshape(-1)
    if dtype == WoqWeightDtype.NF4:
        table = torch.tensor(NF4_DEQUANT_TABLE, dtype=torch.float32, device=qt.device)
        q = table[_unpack_int4(qt).long()]
        z = torch.zeros_like(scales)
    elif dtype == WoqWeightDtype.INT4:
        q = _unpack_int4(qt).float()
        z = zps.reshape(-1) if zps is not None else torch.full_like(scales, 8.0)
    else:
        q = qt.float()
        z = zps.reshape(-1) if zps is not None else torch.zeros_like(scales)
    w = (q - z.unsqueeze(-1)) * scales.unsqueeze(-1)
    if weight_shape is not None:
        w = w[: weight_shape[0], : weight_shape[1]].contiguous()
    return w


def dequantize_per_block(qt, scales, zps: Optional[torch.Tensor], dtype, group_size,
                         weight_shape=None):
    if dtype == WoqWeightDtype.NF4:
        q = torch.tensor(NF4_DEQUANT_TABLE, dtype=torch.float32, device=qt.device)[_unpack_int4(qt).long()]
    else:
        q = _unpack_int4(qt).float() if dtype == WoqWeightDtype.INT4 else qt.float()
    N, K = q.shape
    if scales.dim() > 2:
        scales = scales.squeeze()
    if zps is None:
        zps = torch.full_like(scales, 8.0 if dtype == WoqWeightDtype.INT4 else 0.0)
    elif zps.dim() > 2:
        zps = zps.squeeze()
    s = scales.repeat_interleave(group_size, dim=1)[:, :K]
    z = zps.repeat_interleave(group_size, dim=1)[:, :K]
    w = (q - z) * s
    if weight_shape is not None:
        w = w[: weight_shape[0], : weight_shape[1]].contiguous()
    return w
