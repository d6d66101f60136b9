"""B200-native weight-only-quantised linear: the reference's Python surface for this path
(quantization qconfig, WeightOnlyQuantizedLinear, llm.quantization, llm.optimize, fused-epilogue
modules) over libwoq_b200.so."""
from . import _capi  # noqa: F401
from . import quantization  # noqa: F401
from . import nn  # noqa: F401
from . import llm  # noqa: F401
from . import utils  # noqa: F401
from ._ops import load_ops  # noqa: F401

__all__ = ["_capi", "quantization", "nn", "llm", "load_ops"]
