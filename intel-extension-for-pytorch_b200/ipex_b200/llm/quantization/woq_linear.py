"""ipex.llm.quantization.IPEXWeightOnlyQuantizedLinear: device-keyed front door
(reference: intel_extension_for_pytorch/llm/quantization/woq_linear.py:18-59, which maps
"cpu" to its CPU module; here "cuda" maps to the sm_100a implementation)."""
import torch

from ...nn.modules.weight_only_quantization import WeightOnlyQuantizedLinear
from .utils import QuantDtype, QuantMethod


class IPEXWeightOnlyQuantizedLinear(WeightOnlyQuantizedLinear):
    module_mapping = {"cuda": WeightOnlyQuantizedLinear}

    @classmethod
    def from_weight(cls, qweight, scales, zero_points, in_features, out_features, qconfig=None, bias=None,
                    group_size=-1, g_idx=None, quant_method=QuantMethod.GPTQ_GEMM, dtype=QuantDtype.INT4,
                    **kwargs):
        device_type = "cuda" if (qweight.is_cuda or torch.cuda.is_available()) else qweight.device.type
        assert device_type in cls.module_mapping, (
            f"IPEXWeightOnlyQuantizedLinear.from_weight: no implementation for device {device_type}")
        impl = cls.module_mapping[device_type]
        return impl.from_weight(qweight, scales, zero_points, in_features, out_features, qconfig, bias,
                                group_size, g_idx, quant_method, dtype, **kwargs)
