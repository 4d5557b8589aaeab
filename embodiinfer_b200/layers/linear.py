"""Quantised-linear configuration and the method/backend registry.

Mirror of embodiinfer/layers/linear.py:17-328 for the FP8 and NVFP4 methods: the same config
dataclasses and parsers, the same ``f"{method}_{backend}"`` naming, the same selection order and
error behaviour.  ``fp8_native`` and ``nvfp4_native`` resolve to the sm_100a kernels of this
package.  The ``*_torch`` names are accepted by the parsers (recipes load unchanged) but there is
deliberately no CPU or weight-only fallback behind them: resolving to ``torch`` raises.
"""

from __future__ import annotations

import fnmatch
import importlib
from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Any, Protocol, TypeAlias

import torch

_FP8_BACKENDS = frozenset({"auto", "native", "triton", "torch"})
_NVFP4_BACKENDS = frozenset({"auto", "native", "torch"})
_SCALING_SCHEMES = frozenset({"auto", "channelwise", "tensorwise"})


def _matches(patterns: tuple[str, ...], name: str) -> bool:
    return any(fnmatch.fnmatchcase(name, pattern) for pattern in patterns)


@dataclass(frozen=True)
class FP8Config:
    """FP8 W8A8 policy (embodiinfer/layers/linear.py:23-47)."""

    activation_scheme: str = "dynamic"
    ignored_layers: tuple[str, ...] = ()
    backend: str = "auto"
    scaling_scheme: str = "auto"

    def __post_init__(self) -> None:
        if self.activation_scheme != "dynamic":
            raise ValueError("EmbodiInfer online FP8 currently supports activation_scheme='dynamic' only")
        if self.backend not in _FP8_BACKENDS:
            raise ValueError(f"unsupported FP8 backend {self.backend!r}; expected one of {sorted(_FP8_BACKENDS)}")
        if self.scaling_scheme not in _SCALING_SCHEMES:
            raise ValueError(
                f"unsupported FP8 scaling_scheme {self.scaling_scheme!r}; expected one of {sorted(_SCALING_SCHEMES)}"
            )

    def is_ignored(self, name: str) -> bool:
        return _matches(self.ignored_layers, name)


@dataclass(frozen=True)
class NVFP4Config:
    """NVFP4 W4A4 policy (embodiinfer/layers/linear.py:150-168)."""

    activation_scheme: str = "dynamic"
    ignored_layers: tuple[str, ...] = ()
    backend: str = "auto"

    def __post_init__(self) -> None:
        if self.activation_scheme != "dynamic":
            raise ValueError("EmbodiInfer NVFP4 currently supports activation_scheme='dynamic' only")
        if self.backend not in _NVFP4_BACKENDS:
            raise ValueError(
                f"unsupported NVFP4 backend {self.backend!r}; expected one of {sorted(_NVFP4_BACKENDS)}"
            )

    def is_ignored(self, name: str) -> bool:
        return _matches(self.ignored_layers, name)


QuantizationConfig: TypeAlias = FP8Config | NVFP4Config


def _parse_mapping(value: Mapping[str, Any], method: str, allowed: set[str]) -> dict[str, Any]:
    named = str(value.get("method", value.get("quant_method", method))).lower()
    if named != method:
        raise ValueError(f"unsupported quantization method {named!r}")
    ignored = value.get("ignored_layers", ())
    if isinstance(ignored, str) or not isinstance(ignored, Sequence):
        raise TypeError("ignored_layers must be a sequence of glob patterns")
    unknown = set(value) - allowed
    if unknown:
        raise TypeError(f"unknown {method.upper()} config fields: {', '.join(sorted(unknown))}")
    return {
        "activation_scheme": str(value.get("activation_scheme", "dynamic")).lower(),
        "ignored_layers": tuple(str(pattern) for pattern in ignored),
        "backend": str(value.get("backend", "auto")).lower(),
    }


def parse_fp8_config(value: str | Mapping[str, Any] | FP8Config | None) -> FP8Config | None:
    """``None`` | ``"fp8"`` | mapping | config -> :class:`FP8Config` (linear.py:50-84)."""
    if value is None or isinstance(value, FP8Config):
        return value
    if isinstance(value, str):
        if value.lower() != "fp8":
            raise ValueError("quantization must be None, 'fp8', or an FP8 config mapping")
        return FP8Config()
    if not isinstance(value, Mapping):
        raise TypeError("quantization must be None, 'fp8', an FP8Config, or a mapping")
    fields = _parse_mapping(
        value, "fp8", {"method", "quant_method", "activation_scheme", "ignored_layers", "backend", "scaling_scheme"}
    )
    return FP8Config(scaling_scheme=str(value.get("scaling_scheme", "auto")).lower(), **fields)


def parse_nvfp4_config(value: str | Mapping[str, Any] | NVFP4Config | None) -> NVFP4Config | None:
    """``None`` | ``"nvfp4"`` | mapping | config -> :class:`NVFP4Config` (linear.py:171-204)."""
    if value is None or isinstance(value, NVFP4Config):
        return value
    if isinstance(value, str):
        if value.lower() != "nvfp4":
            raise ValueError("quantization must be None, 'nvfp4', or an NVFP4 config mapping")
        return NVFP4Config()
    if not isinstance(value, Mapping):
        raise TypeError("quantization must be None, 'nvfp4', an NVFP4Config, or a mapping")
    return NVFP4Config(
        **_parse_mapping(value, "nvfp4", {"method", "quant_method", "activation_scheme", "ignored_layers", "backend"})
    )


def parse_quantization_config(
    value: str | Mapping[str, Any] | QuantizationConfig | None,
) -> QuantizationConfig | None:
    """Dispatch on the method name (linear.py:210-225); INT8 is outside this package's path."""
    if value is None or isinstance(value, (FP8Config, NVFP4Config)):
        return value
    method = value if isinstance(value, str) else value.get("method", value.get("quant_method", "fp8"))
    method = str(method).lower()
    if method == "fp8":
        return parse_fp8_config(value)
    if method == "nvfp4":
        return parse_nvfp4_config(value)
    raise ValueError(f"unsupported quantization method {method!r}")


class LinearBackend(Protocol):
    """``kernel(inputs, weight, weight_scale, bias=None, **metadata) -> [..., N]`` (linear.py:228-240)."""

    def __call__(
        self,
        inputs: torch.Tensor,
        weight: torch.Tensor,
        weight_scale: torch.Tensor,
        bias: torch.Tensor | None = None,
        **metadata: torch.Tensor,
    ) -> torch.Tensor: ...


class LinearCapability(Protocol):
    """``capability(inputs, weight, weight_scale) -> (available, reason)`` (linear.py:243-250)."""

    def __call__(
        self, inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor
    ) -> tuple[bool, str | None]: ...


_REGISTRY: dict[str, tuple[LinearBackend, LinearCapability | None]] = {}
_LAZY_REGISTRY: dict[str, tuple[str, str, str | None]] = {}


def register_linear(name: str, kernel: LinearBackend, capability: LinearCapability | None = None) -> None:
    if name in _REGISTRY or name in _LAZY_REGISTRY:
        raise ValueError(f"linear backend {name!r} is already registered")
    _REGISTRY[name] = (kernel, capability)


def register_lazy_linear(name: str, module: str, kernel: str, capability: str | None = None) -> None:
    if name in _REGISTRY or name in _LAZY_REGISTRY:
        raise ValueError(f"linear backend {name!r} is already registered")
    _LAZY_REGISTRY[name] = (module, kernel, capability)


def _resolve(name: str) -> tuple[LinearBackend, LinearCapability | None]:
    entry = _REGISTRY.get(name)
    if entry is not None:
        return entry
    if name not in _LAZY_REGISTRY:
        raise ValueError(f"unknown linear backend {name!r}")
    module_name, kernel, capability = _LAZY_REGISTRY[name]
    module = importlib.import_module(module_name)
    entry = (getattr(module, kernel), getattr(module, capability) if capability else None)
    _REGISTRY[name] = entry
    return entry


def get_linear_backend(name: str) -> LinearBackend:
    return _resolve(name)[0]


def resolve_linear_backend(
    method: str, backend: str, inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor
) -> str:
    """Pick the backend name for one call (linear.py:288-314).

    ``"torch"`` is still returned for ``backend == "torch"`` or CPU inputs, as in the reference; the
    kernel registered under that name here raises, because this package ships no fallback.
    """
    if method not in {"fp8", "nvfp4"}:
        raise ValueError(f"unsupported quantization method {method!r}")
    if backend == "torch" or not inputs.is_cuda:
        return "torch"
    if backend == "auto":
        candidates = ("native", "triton", "torch") if method == "fp8" else ("native", "torch")
    else:
        candidates = (backend,)
    reason = None
    for candidate in candidates:
        name = f"{method}_{candidate}"
        if name not in _REGISTRY and name not in _LAZY_REGISTRY:
            reason = f"the {method} {candidate} backend is not part of this build"
            continue
        _, capability = _resolve(name)
        available, reason = capability(inputs, weight, weight_scale) if capability else (True, None)
        if available:
            return candidate
    raise RuntimeError(reason or f"the requested {method} {backend} backend is unavailable")


_NATIVE = "embodiinfer_b200.backend.linear"
for _method in ("fp8", "nvfp4"):
    register_lazy_linear(f"{_method}_native", _NATIVE, f"{_method}_native_linear", f"{_method}_native_capability")
    register_lazy_linear(f"{_method}_torch", _NATIVE, "no_fallback_linear", "no_fallback_capability")
