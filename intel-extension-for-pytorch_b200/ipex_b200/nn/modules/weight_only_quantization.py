"""WeightOnlyQuantizedLinear and its tensor-parallel variant on CUDA.

Same classes, constructors, class methods and attributes as the reference
(intel_extension_for_pytorch/nn/modules/weight_only_quantization.py), so code written against
`ipex.nn.modules.WeightOnlyQuantizedLinear` / `ipex.llm.quantization.IPEXWeightOnlyQuantizedLinear`
keeps working; the operators they call are registered for the CUDA dispatch key by the
extension in this package and run the sm_100a kernels."""
from enum import IntEnum
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from ..._ops import load_ops
from ..._enums import QuantDtype, QuantMethod
from ..utils._model_convert import _convert_awq_scales_qzeros, _convert_gptq_scales_qzeros
from ...quantization import (QConfigWoq, WoqActQuantMode, WoqLowpMode, WoqWeightDtype,
                            WoqWeightQScheme, quantize_per_block, quantize_per_channel)
from ...quantization._qconfig import (WOQ_ACT_QUANT_MODE_TO_STR, WOQ_DTYPE_TO_STR,
                                     WOQ_LOWP_MODE_TO_STR, WOQ_QSCHEME_TO_STR)


class WoqWeightFormat(IntEnum):
    PLAIN_FORMAT = 0
    GPTQ_FORMAT = 1
    AWQ_FORMAT = 2


def _cuda(t: Optional[torch.Tensor], device=None):
    if t is None or t.is_cuda:
        return t
    return t.to(device if device is not None else torch.device("cuda", torch.cuda.current_device()))


def _gptq_qweight_to_plain(qweight: torch.Tensor) -> torch.Tensor:
    """AutoGPTQ qweight [K/8, N] int32 (nibble i of a word = input channel 8 r + i) -> plain [N, K/2]
    uint8 with the even input channel in the low nibble."""
    shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
    q = (qweight.unsqueeze(1) >> shifts.view(1, 8, 1)) & 0xF          # [K/8, 8, N]
    q = q.reshape(-1, qweight.shape[1]).t().contiguous().to(torch.uint8)  # [N, K]
    return (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()


class WeightOnlyQuantizedLinear(nn.Module):
    r"""A weight-only quantized (WOQ) linear module with floating point tensors as inputs and
    outputs.  The weight lives on the GPU in the kernels' tiled layout."""

    def __init__(self, in_features, out_features, bias_=True, dtype=WoqWeightDtype.INT8):
        super().__init__()
        load_ops()
        self.in_features = in_features
        self.out_features = out_features
        self.bias = bias_
        self.dtype = dtype
        self.weight = None  # plain-format quantised weight, for queries of dtype / shape
        self._op_context = None
        self._lowp_mode = 0
        self._act_quant_mode = 0
        self._group_size = -1
        self._cache_weight_for_large_batch = False
        self._weight_qscheme = WoqWeightQScheme.ASYMMETRIC

    def pre_ipex_gemm(self, input):
        return input

    def post_ipex_gemm(self, output):
        return output

    def forward(self, x):
        x = self.pre_ipex_gemm(x)
        Y = torch.ops.torch_ipex.ipex_woq_linear(x, self._op_context.get_data_handle())
        return self.post_ipex_gemm(Y)

    def _get_name(self):
        return "WeightOnlyQuantizedLinear"

    def extra_repr(self):
        return (
            "in_features={}, out_features={}, dtype={}, bias={}, lowp_mode={}, act_quant_mode={}, "
            "group_size={}, cache_weight_for_large_batch={}, weight_qscheme={}".format(
                self.in_features, self.out_features, WOQ_DTYPE_TO_STR[self.dtype], self.bias,
                WOQ_LOWP_MODE_TO_STR[self._lowp_mode], WOQ_ACT_QUANT_MODE_TO_STR[self._act_quant_mode],
                self._group_size, self._cache_weight_for_large_batch,
                WOQ_QSCHEME_TO_STR[self._weight_qscheme]))

    # ---- constructors ---------------------------------------------------------------------
    @classmethod
    def from_float(cls, mod, scales=None, zero_points=None):
        r"""Create a weight-only quantized module from a float nn.Linear carrying a WOQ qconfig."""
        assert isinstance(mod, nn.Linear) or hasattr(mod, "weight"), (
            "WeightOnlyQuantizedLinear.from_float only works for nn.Linear or its subclasses, "
            f"but found {type(mod)}")
        assert hasattr(mod, "qconfig"), "Input float module must have qconfig defined"
        qconfig = mod.qconfig
        if qconfig is None or not isinstance(qconfig, QConfigWoq):
            return mod
        lowp_mode = qconfig.lowp_mode
        act_quant_mode = qconfig.act_quant_mode
        dtype = qconfig.weight_dtype
        group_size = qconfig.group_size
        sym_quant = qconfig.weight_qscheme == WoqWeightQScheme.SYMMETRIC
        if dtype == WoqWeightDtype.NF4 or (dtype == WoqWeightDtype.INT8 and lowp_mode == WoqLowpMode.INT8):
            assert sym_quant is True, "WOQ NF4 and INT8 with lowp-mode 3 must use symmetric quantization"
        w = _cuda(mod.weight.detach())
        if group_size == -1:
            qweight, scales, zero_points = quantize_per_channel(w, dtype, scales, zero_points, sym_quant)
        else:
            qweight, scales, zero_points = quantize_per_block(w, dtype, group_size, scales, zero_points, sym_quant)
        if not hasattr(mod, "in_features"):
            mod.in_features = mod.weight.size()[1]
        if not hasattr(mod, "out_features"):
            mod.out_features = mod.weight.size()[0]
        cache = qconfig.cache_weight_for_large_batch and lowp_mode in (2, 3)
        qlinear = cls._init_cls(mod, dtype, qweight, scales, zero_points, None, None, group_size,
                                lowp_mode, act_quant_mode, cache, False)
        del qweight
        mod.weight = torch.nn.Parameter()
        return qlinear

    @classmethod
    def from_float_and_qweight(cls, mod, qweight, dtype, scales, zero_points, bias=None, group_size=-1,
                               g_idx=None, weight_format=WoqWeightFormat.PLAIN_FORMAT):
        r"""Create a WOQ module from a float module and an already quantised weight."""
        assert hasattr(mod, "qconfig"), "Input float module must have qconfig defined"
        lowp_mode, act_quant_mode, cache = 0, 0, False
        if mod.qconfig is not None:
            lowp_mode = getattr(mod.qconfig, "lowp_mode", 0)
            act_quant_mode = getattr(mod.qconfig, "act_quant_mode", 0)
            cache = getattr(mod.qconfig, "cache_weight_for_large_batch", False) and lowp_mode in (2, 3)
        supported = [torch.int32, torch.uint8, torch.int8, torch.quint4x2]
        assert qweight.dtype in supported, (
            "Data type of quantized weight should be in {}, but got: {}".format(supported, qweight.dtype))
        if not hasattr(mod, "in_features"):
            mod.in_features = mod.weight.size()[1]
        if not hasattr(mod, "out_features"):
            mod.out_features = mod.weight.size()[0]
        if group_size < 0:
            scales = scales.squeeze()
            if zero_points is not None:
                zero_points = zero_points.squeeze()
        qlinear = cls._init_cls(mod, dtype, qweight, scales, zero_points, bias, g_idx, group_size,
                                lowp_mode, act_quant_mode, cache, dtype == WoqWeightDtype.INT4, weight_format)
        mod.weight = torch.nn.Parameter()
        return qlinear

    @classmethod
    def from_float_and_int4_weight(cls, mod, qweight, scales, zero_points, bias=None, group_size=-1,
                                   g_idx=None, weight_format=WoqWeightFormat.PLAIN_FORMAT):
        print("[WARNING] from_float_and_int4_weight() is deprecated. Please use from_float_and_qweight() instead.")
        return cls.from_float_and_qweight(mod, qweight, WoqWeightDtype.INT4, scales, zero_points, bias,
                                          group_size, g_idx, weight_format)

    @classmethod
    def from_int4_weight(cls, qweight, scales, zero_points, in_features, out_features, quant_method,
                         qconfig=None, bias=None, group_size=-1, g_idx=None):
        r"""Create a WOQ module from an INT4 checkpoint weight (AutoAWQ or AutoGPTQ layout)."""
        lowp_mode = WoqLowpMode.BF16
        act_quant_mode = WoqActQuantMode.PER_IC_BLOCK
        cache = False
        if qconfig is not None and hasattr(qconfig, "global_qconfig"):
            g = qconfig.global_qconfig
            lowp_mode = getattr(g, "lowp_mode", lowp_mode)
            act_quant_mode = getattr(g, "act_quant_mode", act_quant_mode)
            cache = getattr(g, "cache_weight_for_large_batch", False) and lowp_mode in (
                WoqLowpMode.BF16, WoqLowpMode.INT8)
        assert qweight.dtype in (torch.int32, torch.uint8, torch.quint4x2), (
            "Data type of int4 weight should be in [int32, uint8, quint4x2], but got: {}".format(qweight.dtype))
        qlinear = cls(in_features, out_features, dtype=WoqWeightDtype.INT4)
        weight_format = WoqWeightFormat.PLAIN_FORMAT
        if quant_method == QuantMethod.AWQ_GEMM:
            scales, zero_points = _convert_awq_scales_qzeros(scales, zero_points)
            weight_format = WoqWeightFormat.AWQ_FORMAT
        elif quant_method == QuantMethod.GPTQ_GEMM:
            scales, zero_points = _convert_gptq_scales_qzeros(scales, zero_points)
            weight_format = WoqWeightFormat.GPTQ_FORMAT
            if g_idx is not None:
                # act-order: the context shuffles the input channels of a plain weight
                qweight = _gptq_qweight_to_plain(_cuda(qweight))
                weight_format = WoqWeightFormat.PLAIN_FORMAT
        if bias is not None and torch.count_nonzero(bias) == 0:
            bias = None
        qlinear._op_context = torch.ops.ipex_prepack.weight_only_qlinear_prepack_int4(
            _cuda(qweight), _cuda(scales), _cuda(zero_points), _cuda(bias), _cuda(g_idx), None, group_size,
            int(lowp_mode), int(act_quant_mode), cache, int(weight_format))
        qlinear.weight = qlinear._op_context.get_weight()
        qlinear.bias = bias is not None
        qlinear._lowp_mode = lowp_mode
        qlinear._act_quant_mode = act_quant_mode
        qlinear._group_size = group_size
        qlinear._cache_weight_for_large_batch = cache
        qlinear._weight_qscheme = (WoqWeightQScheme.ASYMMETRIC if zero_points is not None
                                   else WoqWeightQScheme.SYMMETRIC)
        return qlinear

    @classmethod
    def from_weight(cls, qweight: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor,
                    in_features: int, out_features: int, qconfig=None, bias: Optional[torch.Tensor] = None,
                    group_size: int = -1, g_idx: Optional[torch.Tensor] = None,
                    quant_method: QuantMethod = QuantMethod.GPTQ_GEMM, dtype: QuantDtype = QuantDtype.INT4,
                    **kwargs):
        r"""Create a WOQ module from checkpoint tensors (4-bit AWQ or GPTQ)."""
        if quant_method in [QuantMethod.GPTQ_GEMM, QuantMethod.AWQ_GEMM] and dtype == QuantDtype.INT4:
            return cls.from_int4_weight(qweight, scales, zero_points, in_features, out_features, quant_method,
                                        qconfig, bias, group_size, g_idx)
        raise AssertionError("Currently ipex.llm.quantization.IPEXWeightOnlyQuantizedLinear.from_weight() "
                             "supports 4bits with AWQ or GPTQ.")

    @classmethod
    def _init_cls(cls, mod, dtype, qweight, scales, zero_points, bias, g_idx, group_size, lowp_mode,
                  act_quant_mode, cache_weight_for_large_batch, is_from_int4_weight,
                  weight_format=WoqWeightFormat.PLAIN_FORMAT):
        if bias is None and mod.bias is not None:
            bias = mod.bias
        if bias is not None and torch.count_nonzero(bias) == 0:
            bias = None
        bias = None if bias is None else bias.detach()
        qlinear = cls(mod.in_features, mod.out_features, bias is not None, dtype=dtype)
        if is_from_int4_weight:
            qlinear._op_context = torch.ops.ipex_prepack.weight_only_qlinear_prepack_int4(
                _cuda(qweight), _cuda(scales), _cuda(zero_points), _cuda(bias), g_idx, None, group_size,
                int(lowp_mode), int(act_quant_mode), cache_weight_for_large_batch, int(weight_format))
        else:
            qlinear._op_context = torch.ops.ipex_prepack.weight_only_qlinear_prepack(
                _cuda(qweight), int(dtype), [mod.out_features, mod.in_features], _cuda(scales),
                _cuda(zero_points), _cuda(bias), g_idx, None, group_size, int(lowp_mode),
                int(act_quant_mode), cache_weight_for_large_batch)
        qlinear.weight = qlinear._op_context.get_weight()
        qlinear.bias = bias is not None
        qlinear._lowp_mode = lowp_mode
        qlinear._act_quant_mode = act_quant_mode
        qlinear._group_size = group_size
        qlinear._cache_weight_for_large_batch = cache_weight_for_large_batch
        qlinear._weight_qscheme = (WoqWeightQScheme.ASYMMETRIC if zero_points is not None
                                   else WoqWeightQScheme.SYMMETRIC)
        return qlinear


class IpexWoqLinearAllreduce(WeightOnlyQuantizedLinear):
    """Row-parallel WOQ linear: this rank holds a K shard; the partial outputs are summed with an
    all-reduce (NCCL on GPUs) and the bias is added after the reduction
    (reference: nn/modules/weight_only_quantization.py:536-633)."""

    def __init__(self, in_features, out_features, mp_group, bias_value, bias_=True, dtype=WoqWeightDtype.INT8):
        super().__init__(in_features, out_features, bias_, dtype=dtype)
        self.mp_group = mp_group
        self.original_bias = bias_value

    def _get_name(self):
        return "IpexWoqLinearAllreduce"

    @classmethod
    def _init_from_mod(cls, mod, dtype):
        return cls(mod.in_features, mod.out_features, getattr(mod, "mp_group", None), mod.bias,
                   mod.bias is not None, dtype=dtype)

    @classmethod
    def _init_cls(cls, mod, dtype, qweight, scales, zero_points, bias, g_idx, group_size, lowp_mode,
                  act_quant_mode, cache_weight_for_large_batch, is_from_int4_weight,
                  weight_format=WoqWeightFormat.PLAIN_FORMAT):
        qlinear = cls._init_from_mod(mod, dtype)
        if bias is not None:
            qlinear.original_bias = nn.Parameter(bias)
        # the bias is withheld from the packed context: it must be added once, after the reduce
        if is_from_int4_weight:
            qlinear._op_context = torch.ops.ipex_prepack.weight_only_qlinear_prepack_int4(
                _cuda(qweight), _cuda(scales), _cuda(zero_points), None, g_idx, None, group_size,
                int(lowp_mode), int(act_quant_mode), cache_weight_for_large_batch, int(weight_format))
        else:
            qlinear._op_context = torch.ops.ipex_prepack.weight_only_qlinear_prepack(
                _cuda(qweight), int(dtype), [mod.out_features, mod.in_features], _cuda(scales),
                _cuda(zero_points), None, g_idx, None, group_size, int(lowp_mode), int(act_quant_mode),
                cache_weight_for_large_batch)
        qlinear.weight = qlinear._op_context.get_weight()
        qlinear._lowp_mode = lowp_mode
        qlinear._act_quant_mode = act_quant_mode
        qlinear._group_size = group_size
        qlinear._cache_weight_for_large_batch = cache_weight_for_large_batch
        qlinear._weight_qscheme = (WoqWeightQScheme.ASYMMETRIC if zero_points is not None
                                   else WoqWeightQScheme.SYMMETRIC)
        return qlinear

    def post_ipex_gemm(self, output):
        return all_reduce_and_bias_add(self.mp_group, self.original_bias, output)


def all_reduce_and_bias_add(mp_group, original_bias, output):
    """Sum over the tensor-parallel group, then add the bias (reference:
    nn/utils/_weight_prepack.py:139-158)."""
    if dist.is_available() and dist.is_initialized() and (mp_group is not None or dist.get_world_size() > 1):
        dist.all_reduce(output, group=mp_group)
    if original_bias is not None:
        output = output + original_bias.to(output.device, output.dtype)
    return output


IPEXWeightOnlyQuantizedLinear = WeightOnlyQuantizedLinear
