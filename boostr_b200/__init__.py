"""B200-native quantized-linear path behind boostr's QuantTensor / QuantMatmulOps surface."""
from .format import QuantError, QuantFormat  # noqa: F401

__all__ = ["QuantError", "QuantFormat"]
