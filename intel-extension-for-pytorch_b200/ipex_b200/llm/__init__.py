from . import quantization  # noqa: F401
from .frontend import optimize  # noqa: F401
