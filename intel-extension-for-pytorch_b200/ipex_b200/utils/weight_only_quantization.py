"""Load a low-precision checkpoint (GPTQ, AWQ or block-scaled FP8 state dict) into a model whose
nn.Linear modules become weight-only-quantised ones, without ever materialising fp32 weights.

Same entry point, arguments and checkpoint conventions as the reference's
_convert_woq_with_low_precision_checkpoint
(intel_extension_for_pytorch/utils/weight_only_quantization.py:21-375):

  gptq   <name>.qweight [K/8, N] int32, <name>.scales [K/G, N], <name>.qzeros [K/G, N/8] int32
         (stored minus one), optional <name>.g_idx [K] (act-order) and <name>.bias
  awq    <name>.qweight [K, N/8] int32 in AWQ nibble order, <name>.scales [K/G, N],
         <name>.qzeros [K/G, N/8] int32, optional <name>.bias
  fp8    <name>.weight [N, K] float8_e4m3fn (or uint8 bit patterns),
         <name>.weight_scale_inv [ceil(N/bn), K/bk] with quant_config["weight_block_size"] = [bn, bk]

Linears without scales in the checkpoint (lm_head) keep a floating weight taken from it; every
other parameter found in the state dict is copied over.  The DeepSpeed module mapping of the
reference is not part of this build (tensor parallelism goes through IpexWoqLinearAllreduce)."""
import copy

import torch

from ..nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear, WoqWeightFormat
from ..nn.utils._model_convert import _convert_awq_scales_qzeros, _convert_gptq_scales_qzeros, _unpack_int32_cols
from ..quantization import WoqWeightDtype

_KEYS = {
    "gptq": ("qweight", "scales", "qzeros", "bias", "g_idx"),
    "awq": ("qweight", "scales", "qzeros", "bias", "g_idx"),
    "fp8": ("weight", "weight_scale_inv", "qzeros", "bias", "g_idx"),
}


def _gptq_to_plain(qweight, scales, qzeros):
    """GPTQ tensors -> plain [N, K/2] nibbles (even k low), scales / zero points [N, groups]: the
    form an act-order layer needs, because its input channels are shuffled at prepack
    (reference: nn/utils/_model_convert.py _convert_optimum_format_to_desired)."""
    k8, n = qweight.shape
    q = torch.empty((k8 * 8, n), dtype=torch.uint8, device=qweight.device)
    for j in range(8):
        q[j::8] = ((qweight >> (4 * j)) & 0xF).to(torch.uint8)
    q = q.t().contiguous()  # [N, K]
    plain = (q[:, ::2] | (q[:, 1::2] << 4)).contiguous()
    scales, zps = _convert_gptq_scales_qzeros(scales, qzeros)
    return plain, scales, zps


def _get_linear_parameters(attr_name, state_dict, quant_config, desc_act):
    method = quant_config["quant_method"]
    w_key, s_key, z_key, b_key, g_key = (attr_name + "." + k for k in _KEYS[method])
    qweight = state_dict.get(w_key)
    scales = state_dict.get(s_key)
    qzeros = state_dict.get(z_key)
    bias = state_dict.get(b_key)
    g_idx = state_dict.get(g_key)
    group_size, fmt = -1, WoqWeightFormat.PLAIN_FORMAT
    if qweight is None or scales is None:
        return state_dict.get(attr_name + ".weight"), None, None, bias, group_size, None, fmt
    if method == "gptq":
        k = qweight.size(0) * 8
        assert scales.dim() == 2, "Unexpected scales tensor dimension"
        if scales.size(0) != 1:
            group_size = 2 ** (k // scales.size(0) - 1).bit_length()
        if desc_act is False:
            g_idx = None
        if g_idx is not None and group_size > 0:
            dummy = torch.arange(k, device=g_idx.device, dtype=g_idx.dtype) // group_size
            if torch.equal(g_idx, dummy) or g_idx.count_nonzero() == 0:
                g_idx = None  # a g_idx that only restates the natural order
        if g_idx is not None:
            qweight, scales, qzeros = _gptq_to_plain(qweight, scales, qzeros)
        else:
            scales, qzeros = _convert_gptq_scales_qzeros(scales, qzeros)
            fmt = WoqWeightFormat.GPTQ_FORMAT
    elif method == "awq":
        assert qweight.size(0) % scales.size(0) == 0, "Uneven group sizes are not supported"
        group_size = qweight.size(0) // scales.size(0)
        scales, qzeros = _convert_awq_scales_qzeros(scales, qzeros)
        fmt, g_idx = WoqWeightFormat.AWQ_FORMAT, None
    else:  # fp8: one scale per [bn, bk] block of the weight -> per row and K group of bk
        bn, bk = quant_config["weight_block_size"]
        assert qweight.size(1) % bk == 0, f"weight width is not divisible by {bk}, got {tuple(qweight.shape)}"
        if qweight.dtype != torch.uint8:
            qweight = qweight.view(torch.uint8)
        if scales.size(0) != qweight.size(0):
            assert (qweight.size(0) + bn - 1) // bn == scales.size(0), (
                f"WOQ FP8 got misaligned shapes of weight and scales: {tuple(qweight.shape)}, {tuple(scales.shape)}")
            scales = torch.repeat_interleave(scales, bn, 0)[: qweight.size(0)].contiguous()
        group_size, qzeros, g_idx = bk, None, None
    return qweight, scales, qzeros, bias, group_size, g_idx, fmt


def _convert_woq_with_low_precision_checkpoint(model, qconfig_mapping, low_precision_checkpoint, quant_config,
                                               inplace=True):
    assert isinstance(low_precision_checkpoint, dict), "low_precision_checkpoint should be a state_dict"
    method = quant_config["quant_method"]
    assert method in _KEYS, f"{method} is not supported, quantization_method choice in [`gptq`, `awq`, `fp8`]."
    target = WoqWeightDtype.FP8 if method == "fp8" else WoqWeightDtype.INT4
    forced_group = quant_config.get("group_size", None)
    desc_act = quant_config.get("desc_act", None)
    state_dict = low_precision_checkpoint
    w_key, s_key = _KEYS[method][:2]
    assert any(k.endswith("." + w_key) for k in state_dict) and any(k.endswith("." + s_key) for k in state_dict), (
        "Error: Format of checkpoint and config do not match")
    qconfig = getattr(qconfig_mapping, "global_qconfig", qconfig_mapping)

    def convert(mod, attr_name):
        if isinstance(mod, torch.nn.Linear):
            mod.qconfig = qconfig
            weight, scales, qzeros, bias, group_size, g_idx, fmt = _get_linear_parameters(
                attr_name, state_dict, quant_config, desc_act)
            if forced_group is not None and scales is not None and method != "fp8":
                group_size = forced_group
            if scales is None:  # a layer the checkpoint keeps in floating point (lm_head)
                if weight is not None and weight.is_floating_point():
                    mod.weight = torch.nn.Parameter(weight)
                    if bias is not None and isinstance(mod.bias, torch.nn.Parameter):
                        mod.bias = torch.nn.Parameter(bias)
                return mod
            return WeightOnlyQuantizedLinear.from_float_and_qweight(
                mod, weight, target, scales, qzeros, bias, group_size=group_size, g_idx=g_idx, weight_format=fmt)
        if isinstance(getattr(mod, "weight", None), torch.nn.Parameter):
            mod.weight = torch.nn.Parameter(state_dict.get(attr_name + ".weight", mod.weight.data))
            if isinstance(getattr(mod, "bias", None), torch.nn.Parameter):
                mod.bias = torch.nn.Parameter(state_dict.get(attr_name + ".bias", mod.bias.data))
            return mod
        for name, child in list(mod.named_children()):
            setattr(mod, name, convert(child, attr_name + "." + name if attr_name else name))
        return mod

    return convert(model if inplace else copy.deepcopy(model), "")
