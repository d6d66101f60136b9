from ..._enums import QuantDtype, QuantMethod  # noqa: F401
