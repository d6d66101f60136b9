"""B200-native weight-only-quantised linear: Python surface over libwoq_b200.so."""
from . import _capi  # noqa: F401

__all__ = ["_capi"]
