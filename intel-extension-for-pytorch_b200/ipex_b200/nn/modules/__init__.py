from .weight_only_quantization import (  # noqa: F401
    IPEXWeightOnlyQuantizedLinear,
    IpexWoqLinearAllreduce,
    WeightOnlyQuantizedLinear,
    WoqWeightFormat,
)
