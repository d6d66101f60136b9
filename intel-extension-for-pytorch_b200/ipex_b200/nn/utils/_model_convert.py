"""Checkpoint-layout helpers for GPTQ / AWQ INT4 weights: bring scales and packed zero points to
[N, groups] (reference: intel_extension_for_pytorch/nn/utils/_model_convert.py:187-330)."""
import torch

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _unpack_int32_cols(q: torch.Tensor, order=None) -> torch.Tensor:
    """[R, C/8] int32 -> [R, C]; nibble j of a word is column 8*c + (order[j] if order else j)."""
    R, C8 = q.shape
    out = torch.empty((R, C8 * 8), dtype=torch.int32, device=q.device)
    for j in range(8):
        col = order[j] if order is not None else j
        out[:, col::8] = (q >> (4 * j)) & 0xF
    return out


def _convert_gptq_scales_qzeros(scales, qzeros, inplace=True):
    """GPTQ: scales [groups, N], qzeros [groups, N/8] stored minus one ->
    scales [N, groups], zero points [N, groups] (plus one, wrapped to 4 bits)."""
    scales = scales.t().contiguous()
    if qzeros is None:
        return scales, None
    zp = _unpack_int32_cols(qzeros).t().contiguous() + 1
    zp = torch.where(zp > 15, torch.zeros_like(zp), zp)
    return scales, zp


def _convert_awq_scales_qzeros(scales, qzeros, inplace=True):
    """AWQ: scales [groups, N], qzeros [groups, N/8] in AWQ nibble order ->
    scales [N, groups], zero points [N, groups]."""
    scales = scales.t().contiguous()
    if qzeros is None:
        return scales, None
    return scales, _unpack_int32_cols(qzeros, AWQ_ORDER).t().contiguous()
