"""Weight bundles ``FP8Linear`` / ``NVFP4Linear``: the state-dict layout of the reference, unchanged.

Mirror of embodiinfer/models/linear.py:28-209, 303-465 (the INT8 bundle is outside this path):
  FP8Linear    weight uint8 [N, K] (e4m3 payload), weight_scale fp32 () or [N], bias
  NVFP4Linear  weight uint8 [N, K/2], weight_scale uint8 [N, K/16] (e4m3 payload),
               weight_scale_blocked uint8 (128x4-tile order), weight_global_scale fp32 (),
               quantization_thresholds fp32 [7], bias
so a checkpoint quantised by either implementation loads into the other.  ``forward`` resolves
``{method}_{backend}`` through ``embodiinfer_b200.layers.linear`` on every call, like the reference.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from collections.abc import Callable
from typing import Any, ClassVar

import torch
from torch import nn

from . import weights as W
from .layers.linear import FP8Config, NVFP4Config, QuantizationConfig, get_linear_backend, resolve_linear_backend


class QuantizedLinear(nn.Module, ABC):
    """Common interface of the quantised projections."""

    quantization_method: ClassVar[str]

    def _apply(self, fn: Callable[[torch.Tensor], torch.Tensor], recurse: bool = True) -> "QuantizedLinear":
        """Move/cast the module but keep fp32 metadata (scales, thresholds) in fp32.

        ``policy.to(torch.bfloat16)`` must not round the scales: they are re-materialised from the
        fp32 originals on the new device (models/linear.py:41-60).
        """
        keep = {name: value for name, value in self._buffers.items() if value is not None and value.dtype == torch.float32}
        probe = torch.empty(0, device=self.weight.device, dtype=self.compute_dtype)
        result = super()._apply(fn, recurse=recurse)
        for name, original in keep.items():
            moved = self._buffers[name]
            if moved.dtype != torch.float32:
                self._buffers[name] = original.to(device=moved.device)
        self.compute_dtype = fn(probe).dtype
        return result

    @classmethod
    @abstractmethod
    def from_linear(cls, linear: nn.Module, config: Any) -> "QuantizedLinear": ...

    @classmethod
    @abstractmethod
    def pack(cls, linears: tuple["QuantizedLinear", ...]) -> "QuantizedLinear": ...

    @property
    def quantized_weight(self) -> torch.Tensor:
        return self.weight

    def _linear_metadata(self) -> dict[str, torch.Tensor]:
        return {}

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if inputs.shape[-1] != self.in_features:
            raise ValueError(f"{type(self).__name__} expected K={self.in_features}, got {inputs.shape[-1]}")
        backend = resolve_linear_backend(
            self.quantization_method, self.backend, inputs, self.quantized_weight, self.weight_scale
        )
        kernel = get_linear_backend(f"{self.quantization_method}_{backend}")
        return kernel(inputs, self.quantized_weight, self.weight_scale, self.bias, **self._linear_metadata())

    def extra_repr(self) -> str:
        return (
            f"in_features={self.in_features}, out_features={self.out_features}, "
            f"bias={self.bias is not None}, backend={self.backend!r}"
        )

    def _finish(self, bias, split_sizes) -> None:
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = bias
        if split_sizes is not None:
            self.split_sizes = split_sizes


def _source_weight(linear: nn.Module, method: str) -> torch.Tensor:
    weight = getattr(linear, "weight", None)
    if not isinstance(weight, torch.Tensor) or weight.ndim != 2:
        raise TypeError(f"cannot {method}-quantize {type(linear).__name__} without a matrix weight")
    return weight


def _split_sizes(linear: nn.Module) -> tuple[int, ...] | None:
    sizes = getattr(linear, "split_sizes", None)
    return None if sizes is None else tuple(sizes)


class FP8Linear(QuantizedLinear):
    quantization_method = "fp8"

    def __init__(
        self,
        weight: torch.Tensor,
        weight_scale: torch.Tensor,
        bias: nn.Parameter | None,
        *,
        compute_dtype: torch.dtype,
        backend: str = "auto",
        split_sizes: tuple[int, ...] | None = None,
    ) -> None:
        super().__init__()
        if weight.ndim != 2 or weight_scale.shape not in ((), (weight.shape[0],)):
            raise ValueError("FP8Linear expects weight [N, K] and scalar or per-channel scale")
        if weight.dtype == torch.float8_e4m3fn:
            weight = weight.view(torch.uint8)
        elif weight.dtype != torch.uint8:
            raise ValueError("FP8Linear weight must contain E4M3 data")
        self.out_features, self.in_features = int(weight.shape[0]), int(weight.shape[1])
        self.compute_dtype, self.backend = compute_dtype, backend
        self.weight = nn.Parameter(weight, requires_grad=False)
        self.register_buffer("weight_scale", weight_scale)
        self._finish(bias, split_sizes)

    @property
    def quantized_weight(self) -> torch.Tensor:
        return self.weight.view(torch.float8_e4m3fn)

    @classmethod
    def from_linear(cls, linear: nn.Module, config: FP8Config) -> "FP8Linear":
        weight = _source_weight(linear, "FP8")
        codes, scale = W.fp8_quantize_weight(
            weight.detach(), backend=config.backend, scaling_scheme=config.scaling_scheme
        )
        module = cls(codes, scale, getattr(linear, "bias", None), compute_dtype=weight.dtype, backend=config.backend,
                     split_sizes=_split_sizes(linear))
        return module.train(linear.training)

    @classmethod
    def pack(cls, linears: tuple["FP8Linear", ...]) -> "FP8Linear":
        """Concatenate projections that share an input; tensorwise members are requantised to one scale
        and afterwards view the packed storage (models/linear.py:156-202)."""
        if not linears:
            raise ValueError("cannot pack an empty FP8 linear sequence")
        first = linears[0]
        for other in linears:
            if (other.in_features != first.in_features or other.compute_dtype != first.compute_dtype
                    or other.backend != first.backend or other.weight.dtype != first.weight.dtype
                    or other.bias is not None):
                raise ValueError("FP8 fused projections must have matching inputs, dtype, backend, and no bias")
        if first.weight_scale.ndim == 0:
            dense = torch.cat(
                [W.fp8_dequantize_weight(m.quantized_weight.detach(), m.weight_scale, torch.float32) for m in linears]
            )
            codes, scale = W.fp8_quantize_weight(dense, scaling_scheme="tensorwise")
        else:
            codes = torch.cat([m.weight.detach() for m in linears]).contiguous()
            scale = torch.cat([m.weight_scale.detach() for m in linears]).contiguous()
        packed = cls(codes, scale, None, compute_dtype=first.compute_dtype, backend=first.backend,
                     split_sizes=tuple(m.out_features for m in linears))
        packed.train(first.training)
        begin = 0
        for member in linears:
            end = begin + member.out_features
            member.weight = nn.Parameter(packed.weight[begin:end], requires_grad=False)
            member.weight_scale = packed.weight_scale if packed.weight_scale.ndim == 0 else packed.weight_scale[begin:end]
            begin = end
        return packed


class NVFP4Linear(QuantizedLinear):
    quantization_method = "nvfp4"

    def __init__(
        self,
        weight: torch.Tensor,
        weight_scale: torch.Tensor,
        weight_global_scale: torch.Tensor,
        bias: nn.Parameter | None,
        *,
        compute_dtype: torch.dtype,
        backend: str = "auto",
        split_sizes: tuple[int, ...] | None = None,
    ) -> None:
        super().__init__()
        if weight.ndim != 2:
            raise ValueError("NVFP4Linear expects packed weight [N, K/2]")
        if weight_scale.shape != (weight.shape[0], weight.shape[1] // 8):
            raise ValueError("NVFP4Linear expects one weight scale per 16 logical values")
        if weight_scale.dtype == torch.float8_e4m3fn:
            weight_scale = weight_scale.view(torch.uint8)
        elif weight_scale.dtype != torch.uint8:
            raise ValueError("NVFP4Linear weight_scale must contain E4M3 data")
        self.out_features, self.in_features = int(weight.shape[0]), int(weight.shape[1] * 2)
        self.compute_dtype, self.backend = compute_dtype, backend
        self.weight = nn.Parameter(weight, requires_grad=False)
        self.register_buffer("weight_scale", weight_scale)
        self.register_buffer("weight_scale_blocked", W.blocked_scales(weight_scale))
        self.register_buffer("weight_global_scale", weight_global_scale)
        self.register_buffer("quantization_thresholds", W.nvfp4_thresholds(weight))
        self._finish(bias, split_sizes)

    @classmethod
    def from_linear(cls, linear: nn.Module, config: NVFP4Config) -> "NVFP4Linear":
        weight = _source_weight(linear, "NVFP4")
        packed, scale, global_scale = W.nvfp4_quantize_weight(weight.detach())
        module = cls(packed, scale, global_scale, getattr(linear, "bias", None), compute_dtype=weight.dtype,
                     backend=config.backend, split_sizes=_split_sizes(linear))
        return module.train(linear.training)

    @classmethod
    def pack(cls, linears: tuple["NVFP4Linear", ...]) -> "NVFP4Linear":
        """Dequantise, concatenate and requantise under one global scale; members then view the packed
        storage and get their own tiled scale copy (models/linear.py:370-418)."""
        if not linears:
            raise ValueError("cannot pack an empty NVFP4 linear sequence")
        first = linears[0]
        for other in linears:
            if (type(other) is not cls or other.in_features != first.in_features
                    or other.compute_dtype != first.compute_dtype or other.backend != first.backend
                    or other.bias is not None):
                raise ValueError("NVFP4 fused projections must match inputs, dtype, backend, and bias")
        dense = torch.cat(
            [W.nvfp4_dequantize_weight(m.weight.detach(), m.weight_scale, m.weight_global_scale, torch.float32)
             for m in linears]
        )
        codes, scale, global_scale = W.nvfp4_quantize_weight(dense, first.quantization_thresholds)
        packed = cls(codes, scale, global_scale, None, compute_dtype=first.compute_dtype, backend=first.backend,
                     split_sizes=tuple(m.out_features for m in linears))
        packed.train(first.training)
        begin = 0
        for member in linears:
            end = begin + member.out_features
            member.weight = nn.Parameter(packed.weight[begin:end], requires_grad=False)
            member.weight_scale = packed.weight_scale[begin:end]
            member.weight_scale_blocked = W.blocked_scales(member.weight_scale)
            member.weight_global_scale = packed.weight_global_scale
            begin = end
        return packed

    def _linear_metadata(self) -> dict[str, torch.Tensor]:
        return {
            "weight_global_scale": self.weight_global_scale,
            "weight_scale_blocked": self.weight_scale_blocked,
            "quantization_thresholds": self.quantization_thresholds,
        }


def quantize_linear(linear: nn.Module, config: QuantizationConfig) -> QuantizedLinear:
    if isinstance(config, FP8Config):
        return FP8Linear.from_linear(linear, config)
    if isinstance(config, NVFP4Config):
        return NVFP4Linear.from_linear(linear, config)
    raise TypeError(f"unsupported quantization config {type(config).__name__}")


def pack_quantized_linears(linears: tuple[QuantizedLinear, ...]) -> QuantizedLinear:
    if not linears:
        raise ValueError("cannot pack an empty quantized linear sequence")
    kind = type(linears[0])
    if not all(type(member) is kind for member in linears):
        raise ValueError("all packed quantized projections must use the same quantization method")
    return kind.pack(linears)


__all__ = ["QuantizedLinear", "FP8Linear", "NVFP4Linear", "quantize_linear", "pack_quantized_linears"]
