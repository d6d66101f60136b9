"""ipex.llm.optimize for the WOQ path: swap the nn.Linear modules of a model for
WeightOnlyQuantizedLinear according to a weight-only qconfig mapping
(reference: transformers/optimize.py:2074-2295 -> quantization/_quantize.py:436-467 convert()).
Only the weight-only-quantisation branch of the reference's optimize() is provided."""
import copy

import torch
from torch import nn

from ..nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear
from ..quantization import QConfigWoq


def convert(model: nn.Module, qconfig, skip=("lm_head",)):
    """Replace every nn.Linear (except names in `skip`) by its weight-only-quantised version."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and name not in skip:
            child.qconfig = qconfig
            setattr(model, name, WeightOnlyQuantizedLinear.from_float(child))
        else:
            convert(child, qconfig, skip)
    return model


def optimize(model, dtype=torch.bfloat16, quantization_config=None, inplace=False, device="cuda", **kwargs):
    assert quantization_config is not None, "this build of llm.optimize covers weight-only quantisation"
    qconfig = getattr(quantization_config, "global_qconfig", quantization_config)
    assert isinstance(qconfig, QConfigWoq), "quantization_config must come from get_weight_only_quant_qconfig_mapping"
    if not inplace:
        model = copy.deepcopy(model)
    model = model.eval()
    convert(model, qconfig)
    return model.to(device=device, dtype=dtype)
