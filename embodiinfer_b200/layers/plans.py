"""Plan protocols and the lazy registries of the calibrated ("plan") route.

Mirror of embodiinfer/layers/quantization.py:16-101, embodiinfer/layers/activation.py:13-79 and the
norm + encoder family of embodiinfer/layers/normalization.py:54-107.
A *backend* is constructed once per device through ``BackendRegistry.get``; its ``plan(...)``
allocates every buffer up front so that the per-step calls (``quantize``, ``encode``, ``apply``)
launch kernels only and can be captured into a CUDA graph.
"""

from __future__ import annotations

from collections.abc import Callable, Hashable
from typing import Literal, Protocol

import torch

from .registry import BackendRegistry

Precision = Literal["bf16", "fp8", "nvfp4"]
WorkspaceKey = Hashable


class EncodedActivation(Protocol):
    """What a quantisation plan exposes after ``quantize`` (quantization.py:16-35)."""

    output: torch.Tensor
    scale: torch.Tensor
    scales: torch.Tensor | None
    blocked: torch.Tensor | None


class QuantizationPlanLike(EncodedActivation, Protocol):
    def quantize(self, inputs: torch.Tensor) -> "QuantizationPlanLike": ...


class ActivationQuantizer(Protocol):
    """``plan(inputs, bits, scale=None)``; ``scale=None`` means dynamic per-tensor (quantization.py:38-45)."""

    def plan(self, inputs: torch.Tensor, bits: int, scale: float | None = None) -> QuantizationPlanLike: ...


class ProjectionPlan(Protocol):
    precision: Precision
    maximum: float

    def encode(self, inputs: torch.Tensor) -> EncodedActivation | None: ...

    def apply(self, inputs: torch.Tensor, encoded: EncodedActivation | None) -> torch.Tensor: ...

    def release_scope(self, scope: WorkspaceKey) -> None: ...


class ProjectionBackend(Protocol):
    """``plan(weight, maximum, precision, quantizer, workspace_key)`` (quantization.py:48-81)."""

    def plan(
        self,
        weight: torch.Tensor,
        maximum: float,
        precision: Precision,
        quantizer: ActivationQuantizer | None,
        workspace_key: Callable[[torch.device], WorkspaceKey],
    ) -> ProjectionPlan: ...


class GeluMulPlan(Protocol):
    output: torch.Tensor

    def encode(self, gate: torch.Tensor, up: torch.Tensor) -> "GeluMulPlan": ...


class GeluMulBackend(Protocol):
    """``plan(gate, bits, scale=None)`` -> ``encode(gate, up)`` (activation.py:21-28)."""

    def plan(self, gate: torch.Tensor, bits: int, scale: float | None = None) -> GeluMulPlan: ...


class NormQuantPlanLike(EncodedActivation, Protocol):
    """Fused residual / RMSNorm / encoding with the quantiser's packed layout (normalization.py:54-82)."""

    def normalize(self, inputs: torch.Tensor, *, scale: torch.Tensor | None = None,
                  modulation: torch.Tensor | None = None) -> EncodedActivation: ...

    def residual_normalize(self, inputs: torch.Tensor, update: torch.Tensor, residual_gate: torch.Tensor | None, *,
                           scale: torch.Tensor | None = None, modulation: torch.Tensor | None = None
                           ) -> tuple[torch.Tensor, EncodedActivation, torch.Tensor | None]: ...


class NormQuantBackend(Protocol):
    """``plan(inputs, bits=, calibrated_scale=, adaptive=)`` (normalization.py:85-96)."""

    def plan(self, inputs: torch.Tensor, *, bits: int, calibrated_scale: float, adaptive: bool) -> NormQuantPlanLike: ...


quantization_backends: BackendRegistry[ActivationQuantizer] = BackendRegistry("quantization")
projection_backends: BackendRegistry[ProjectionBackend] = BackendRegistry("projection")
gelu_mul_backends: BackendRegistry[GeluMulBackend] = BackendRegistry("gelu_mul")
norm_quant_backends: BackendRegistry[NormQuantBackend] = BackendRegistry("residual/norm/quantization")

# The reference's plan callers ask for "cuda"; "native" is this package's own name for the same classes.
for _name in ("cuda", "native"):
    quantization_backends.register_lazy(_name, "embodiinfer_b200.backend.quantization", "B200Quantizer")
    gelu_mul_backends.register_lazy(_name, "embodiinfer_b200.backend.activation", "B200GeluMul")
    projection_backends.register_lazy(_name, "embodiinfer_b200.backend.projection", "B200ProjectionBackend")
# The reference's single-pass family ("cuda_reduce": row sums inside the kernel, normalization.py:102-107) is the
# arithmetic b2_norm_quant reproduces; its two-step "cuda_strict" family (torch computes the mean) is reached through
# the plan's ``mean=`` argument.
for _name in ("cuda_reduce", "native"):
    norm_quant_backends.register_lazy(_name, "embodiinfer_b200.backend.norm_quant", "B200NormQuant")
