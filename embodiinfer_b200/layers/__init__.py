"""Registries and configuration contracts (no arithmetic lives here)."""

from .linear import (
    FP8Config,
    NVFP4Config,
    QuantizationConfig,
    get_linear_backend,
    parse_fp8_config,
    parse_nvfp4_config,
    parse_quantization_config,
    register_lazy_linear,
    register_linear,
    resolve_linear_backend,
)
from .plans import gelu_mul_backends, norm_quant_backends, projection_backends, quantization_backends
from .registry import BackendRegistry, OperatorCapabilities, OperatorRequest

__all__ = [
    "BackendRegistry",
    "OperatorCapabilities",
    "OperatorRequest",
    "FP8Config",
    "NVFP4Config",
    "QuantizationConfig",
    "parse_fp8_config",
    "parse_nvfp4_config",
    "parse_quantization_config",
    "register_linear",
    "register_lazy_linear",
    "get_linear_backend",
    "resolve_linear_backend",
    "quantization_backends",
    "projection_backends",
    "gelu_mul_backends",
    "norm_quant_backends",
]
