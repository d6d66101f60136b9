"""Weight-only-quantisation configuration: the enums and the qconfig factory of the reference
(intel_extension_for_pytorch/quantization/_qconfig.py:105-307), same names, values, defaults
and validation."""
import warnings
from collections import namedtuple
from enum import IntEnum

import torch
from torch.ao.quantization import PerChannelMinMaxObserver, PlaceholderObserver, QConfig, QConfigMapping


class WoqLowpMode(IntEnum):
    NONE = 0
    FP16 = 1
    BF16 = 2
    INT8 = 3


class WoqActQuantMode(IntEnum):
    NONE = -1
    PER_TENSOR = 0
    PER_IC_BLOCK = 1  # IC = input channel
    PER_BATCH = 2
    PER_BATCH_IC_BLOCK = 3
    PER_TENSOR_SYM = 4
    PER_IC_BLOCK_SYM = 5
    PER_BATCH_SYM = 6
    PER_BATCH_IC_BLOCK_SYM = 7


class WoqWeightDtype(IntEnum):  # starts at 1 to match the kernel constants
    INT8 = 1
    INT4 = 2
    NF4 = 3
    FP8 = 4


class WoqWeightQScheme(IntEnum):
    UNDEFINED = 0
    ASYMMETRIC = 1
    SYMMETRIC = 2


WOQ_LOWP_MODE_TO_STR = {m: m.name.lower() for m in WoqLowpMode}
WOQ_ACT_QUANT_MODE_TO_STR = {m: m.name.lower() for m in WoqActQuantMode}
WOQ_DTYPE_TO_STR = {m: m.name.lower() for m in WoqWeightDtype}
WOQ_QSCHEME_TO_STR = {m: m.name.lower() for m in WoqWeightQScheme}

QConfigWoq = namedtuple(
    "QConfigWoq",
    [*QConfig._fields, "lowp_mode", "act_quant_mode", "weight_dtype", "group_size",
     "cache_weight_for_large_batch", "weight_qscheme"],
)


def get_weight_only_quant_qconfig_mapping(
    *,
    weight_dtype: int = WoqWeightDtype.INT8,
    lowp_mode: int = WoqLowpMode.NONE,
    act_quant_mode: int = WoqActQuantMode.PER_BATCH_IC_BLOCK_SYM,
    group_size: int = -1,
    weight_qscheme: int = WoqWeightQScheme.UNDEFINED,
):
    """Global QConfigMapping for weight-only quantisation (see the reference docstring for
    the meaning of each argument).  act_quant_mode only matters when lowp_mode is INT8;
    NF4 and INT8-weights-with-INT8-compute are always symmetric."""
    assert group_size == -1 or (group_size > 0 and (group_size & (group_size - 1)) == 0), (
        "Group size must be -1 or a positive power of 2, but got {}".format(group_size))
    if weight_dtype in (torch.qint8, torch.quint4x2):
        weight_dtype = WoqWeightDtype.INT8 if weight_dtype == torch.qint8 else WoqWeightDtype.INT4
        warnings.warn("torch.qint8 and torch.quint4x2 are deprecated for weight only quantization; "
                      "use WoqWeightDtype.INT8 / WoqWeightDtype.INT4.")
    assert weight_dtype in [i.value for i in WoqWeightDtype], (
        f"Invalid weight data type for weight only quantization: {weight_dtype}")
    if lowp_mode != WoqLowpMode.INT8:
        act_quant_mode = WoqActQuantMode.NONE
    must_be_sym = weight_dtype == WoqWeightDtype.NF4 or (
        weight_dtype == WoqWeightDtype.INT8 and lowp_mode == WoqLowpMode.INT8)
    if must_be_sym:
        assert weight_qscheme != WoqWeightQScheme.ASYMMETRIC, (
            "Asymmetric quantization of weight is not supported when (1) weight_dtype is NF4 "
            "or (2) weight_dtype is INT8 and lowp_mode is INT8.")
    if weight_qscheme == WoqWeightQScheme.UNDEFINED:
        weight_qscheme = WoqWeightQScheme.SYMMETRIC if must_be_sym else WoqWeightQScheme.ASYMMETRIC
    qconfig = QConfigWoq(
        activation=PlaceholderObserver.with_args(dtype=torch.float, is_dynamic=False),
        weight=PerChannelMinMaxObserver(),
        lowp_mode=lowp_mode,
        act_quant_mode=act_quant_mode,
        weight_dtype=weight_dtype,
        group_size=group_size,
        cache_weight_for_large_batch=False,
        weight_qscheme=weight_qscheme,
    )
    return QConfigMapping().set_global(qconfig)
