"""Residual update + RMSNorm (offset scale or adaptive modulation) + bf16 rounding + activation encoding in
one launch.

Drop-in for the reference's ``NormQuantReduceFusion`` / ``NormQuantPlan``
(embodiinfer/backend/cuda/norm_quant.py:15-320): same ``plan(inputs, bits=, calibrated_scale=, adaptive=)``,
same plan attributes (``output``, ``scale``, ``scales``, ``blocked``, ``residual``, ``gate``), same
``normalize`` / ``residual_normalize`` signatures, results and validation errors.  The arithmetic and the
order of the row sums are those of the reference's kernels (``b2_norm_quant`` documents them); with
``mean=`` the caller's statistics are used instead, as in the reference's two-step route.
``bits=16`` (not in the reference's plan) returns the normalised bf16 tensor in ``output``.
"""

from __future__ import annotations

import torch

from .. import _native as N
from .. import kernels as K
from ..layers.registry import OperatorCapabilities
from .quantization import B200Quantizer


class B200NormQuant:
    """Plans for [B, T, D] bf16 activations on the backend's device."""

    capabilities = OperatorCapabilities(
        ("cuda",),
        (torch.bfloat16,),
        "torch_rmsnorm_bf16_rounding",
        rank=3,
        width_multiple=64,
        bits=(4, 8),
        minimum_sm_by_bits=((4, (10, 0)),),
        minimum_sm=(10, 0),
    )

    def __init__(self, quantizer: B200Quantizer, norm: object | None = None) -> None:
        """``norm`` is accepted because the reference's callers pass their normalisation backend
        (operators.py:187-189); this kernel computes the statistics itself and does not use it."""
        if not isinstance(quantizer, B200Quantizer):
            raise ValueError("CUDA norm/encoding requires CUDA quantization and strict CUDA normalization")
        self.quantizer, self.device = quantizer, quantizer.device

    def plan(self, inputs: torch.Tensor, *, bits: int, calibrated_scale: float, adaptive: bool) -> "NormQuantPlan":
        """Allocate a fixed-shape calibrated encoder for bf16 [B, T, D] activations."""
        return NormQuantPlan(self, inputs, bits=bits, calibrated_scale=calibrated_scale, adaptive=adaptive)


class NormQuantPlan:
    """Fixed-shape buffers; ``normalize`` and ``residual_normalize`` only launch one kernel (graph-capturable)."""

    def __init__(self, backend: B200NormQuant, inputs: torch.Tensor, *, bits: int, calibrated_scale: float, adaptive: bool) -> None:
        if (
            inputs.device != backend.device
            or inputs.dtype != torch.bfloat16
            or not inputs.is_contiguous()
            or inputs.ndim != 3
            or min(inputs.shape) <= 0
            or inputs.shape[2] % 64
            or bits not in (4, 8, 16)
        ):
            raise ValueError("Norm quantization requires CUDA BF16 [B,T,D], D % 64 == 0, bits 4/8")
        if inputs.shape[2] > 8192:
            raise ValueError("Norm quantization supports widths up to 8192")
        self.backend, self.shape, self.bits, self.adaptive = backend, inputs.shape, bits, adaptive
        if bits == 16:
            self.quantized = None
            self.output = torch.empty_like(inputs)
            self.scale = self.scales = self.blocked = None
        else:
            self.quantized = backend.quantizer.plan(inputs.reshape(-1, inputs.shape[-1]), bits, calibrated_scale)
            self.output, self.scale = self.quantized.output, self.quantized.scale
            self.scales, self.blocked = self.quantized.scales, self.quantized.blocked
        self.residual = torch.empty_like(inputs)
        self.gate = (
            torch.empty((inputs.shape[0], 1, inputs.shape[2]), device=inputs.device, dtype=inputs.dtype) if adaptive else None
        )

    def _validate(self, inputs: torch.Tensor) -> None:
        if (
            inputs.shape != self.shape
            or inputs.device != self.output.device
            or inputs.dtype != torch.bfloat16
            or not inputs.is_contiguous()
        ):
            raise ValueError("Norm quantization input shape, layout, dtype, or device changed")

    def _affine(self, inputs: torch.Tensor, scale: torch.Tensor | None, modulation: torch.Tensor | None) -> None:
        affine = modulation if self.adaptive else scale
        expected = (self.shape[0], self.shape[2] * 3) if self.adaptive else (self.shape[2],)
        if (
            affine is None
            or affine.shape != expected
            or affine.dtype != torch.float32
            or affine.device != inputs.device
            or not affine.is_contiguous()
        ):
            raise ValueError("Norm quantization requires contiguous FP32 scale or raw modulation")

    def _launch(self, inputs, update, update_gate, scale, modulation, mean, residual, flags=0) -> None:
        K.norm_quant(
            inputs, self.output, bits=self.bits, tokens=self.shape[1],
            scale=None if self.adaptive else scale, modulation=modulation if self.adaptive else None,
            update=update, update_gate=update_gate, mean=mean, global_scale=self.scale, residual=residual,
            scales=self.scales if self.bits == 4 else None, blocked=self.blocked if self.bits == 4 else None,
            gate=self.gate, flags=flags,
        )

    def normalize(self, inputs: torch.Tensor, *, scale: torch.Tensor | None = None, modulation: torch.Tensor | None = None,
                  mean: torch.Tensor | None = None) -> "NormQuantPlan":
        """Round the normalised affine result to bf16 in registers, then encode it.

        ``scale``: contiguous fp32 [D] RMSNorm weight without the +1; ``modulation``: contiguous fp32 [B, 3D]
        adaptive scale | shift | gate; ``mean``: optional fp32 [B, T, 1] mean of squares.  Returns this
        workspace, which carries the packed format of a ``QuantizationPlan``."""
        self._validate(inputs)
        self._affine(inputs, scale, modulation)
        if mean is not None and (
            mean.shape != (*self.shape[:2], 1) or mean.dtype != torch.float32 or mean.device != inputs.device
            or not mean.is_contiguous()
        ):
            raise ValueError("Norm quantization requires original FP32 [B,T,1] mean statistics")
        self._launch(inputs, None, None, scale, modulation, mean, None)   # the residual is `inputs` itself: no copy
        return self

    def residual_normalize(self, inputs: torch.Tensor, update: torch.Tensor, residual_gate: torch.Tensor | None, *,
                           scale: torch.Tensor | None = None, modulation: torch.Tensor | None = None,
                           residual_evict_last: bool = False):
        """``residual = bf16(inputs + bf16(update * gate))``, then normalise and encode it.  Returns
        ``(residual, plan, next gate or None)``."""
        self._validate(inputs)
        self._validate(update)
        if residual_gate is not None and (
            residual_gate.shape != (self.shape[0], 1, self.shape[2])
            or residual_gate.dtype != torch.bfloat16
            or residual_gate.device != inputs.device
            or not residual_gate.is_contiguous()
        ):
            raise ValueError("Residual gate must be contiguous CUDA BF16 [B,1,D]")
        self._affine(inputs, scale, modulation)
        self._launch(inputs, update, residual_gate, scale, modulation, None, self.residual,
                     N.NORM_RESIDUAL_EVICT_LAST if residual_evict_last else 0)
        return self.residual, self, self.gate
