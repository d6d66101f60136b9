from .weight_only_quantization import _convert_woq_with_low_precision_checkpoint  # noqa: F401
