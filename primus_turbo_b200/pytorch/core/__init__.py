from . import low_precision
from .backend import BackendType, GlobalBackendManager, PrecisionType
from .quantized_tensor import QuantizedTensor, QuantizedTensorPair

__all__ = ["QuantizedTensor", "QuantizedTensorPair", "BackendType", "GlobalBackendManager", "PrecisionType"]
