from .utils import QuantDtype, QuantMethod  # noqa: F401
from .woq_linear import IPEXWeightOnlyQuantizedLinear  # noqa: F401
