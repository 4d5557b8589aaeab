"""Reusable FP8 / NVFP4 activation-encoding workspaces on the sm_100a kernels.

Drop-in for the reference's ``CudaQuantizer`` / ``QuantizationPlan``
(embodiinfer/backend/cuda/quantization.py:12-166): same capabilities, same plan attributes
(``output``, ``scale``, ``scales``, ``blocked``, ``dynamic``), same validation errors, the CUDA
route's arithmetic (embodiinfer/backend/cuda/csrc/quantize.cu:38-104) bit for bit.
"""

from __future__ import annotations

import math

import torch

from .. import _native as N
from .. import kernels as K
from ..layers.registry import OperatorCapabilities

FP8_BOUND = 448.0
NVFP4_BOUND = 448.0 * 6.0


def blocked_scale_bytes(rows: int, columns: int) -> int:
    """Bytes of the 128x4-tile scale layout for a [rows, columns] matrix (columns % 16 == 0)."""
    return math.ceil(rows / 128) * 128 * math.ceil(columns / 64) * 4


class B200Quantizer:
    """Quantise contiguous bf16 matrices into preallocated FP8 or NVFP4 buffers."""

    capabilities = OperatorCapabilities(
        ("cuda",),
        (torch.bfloat16,),
        "rounded_bf16_encoding",
        rank=2,
        width_multiple=64,
        bits=(4, 8),
        minimum_sm_by_bits=((4, (10, 0)),),
        minimum_sm=(10, 0),
    )

    def __init__(self) -> None:
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.library = N.load()

    def plan(self, inputs: torch.Tensor, bits: int, scale: float | None = None) -> "QuantizationPlan":
        """Allocate reusable buffers; omit ``scale`` for per-tensor dynamic quantisation."""
        return QuantizationPlan(self, inputs, bits, scale)

    def rescale(self, output: torch.Tensor, input_scale: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
        """In place ``output * bf16(input_scale * weight_scale)`` in bf16 (quantize.cu:106-114).

        The fused Linear applies this rounding itself (``B2_LINEAR_ROUND_SCALE_BF16``); this method
        exists for callers that hold an unscaled GEMM result and is one elementwise torch multiply.
        """
        if output.device != self.device or input_scale.device != self.device or weight_scale.device != self.device:
            raise ValueError("Quantizer output and scales must share the backend device")
        return output.mul_((input_scale.float() * weight_scale.float()).to(torch.bfloat16))


class QuantizationPlan:
    """Fixed-shape encoding workspace; ``quantize`` only launches kernels (graph-capturable)."""

    def __init__(self, backend: B200Quantizer, inputs: torch.Tensor, bits: int, scale: float | None) -> None:
        if inputs.device != backend.device or inputs.dtype != torch.bfloat16 or not inputs.is_contiguous():
            raise ValueError("CUDA quantization requires contiguous CUDA BF16 inputs")
        if inputs.ndim != 2 or min(inputs.shape) <= 0 or inputs.shape[1] % 64 or bits not in (4, 8):
            raise ValueError("Expected a matrix with K divisible by 64 and bits in {4, 8}")
        if scale is not None and (not math.isfinite(scale) or scale <= 0):
            raise ValueError("A calibrated scale must be finite and positive")
        self.backend, self.bits, self.shape = backend, bits, inputs.shape
        self.dynamic = scale is None
        device = inputs.device
        rows, columns = inputs.shape
        self.scale = torch.tensor(scale or 1.0, device=device, dtype=torch.float32)
        self.scratch = K.new_scale_scratch(device)
        self.output = torch.empty(
            (rows, columns if bits == 8 else columns // 2),
            device=device,
            dtype=torch.float8_e4m3fn if bits == 8 else torch.uint8,
        )
        self.scales = torch.empty((rows, columns // 16), device=device, dtype=torch.float8_e4m3fn)
        # Rows beyond `rows` in the last 128-row tile are never written: zero them once, here.
        self.blocked = torch.zeros(blocked_scale_bytes(rows, columns), device=device, dtype=torch.float8_e4m3fn)

    def quantize(self, inputs: torch.Tensor) -> "QuantizationPlan":
        if inputs.shape != self.shape or not inputs.is_contiguous():
            raise ValueError("Quantization input shape or layout changed")
        if inputs.device != self.output.device or inputs.dtype != torch.bfloat16:
            raise ValueError("Quantization input device or dtype changed")
        if self.dynamic:
            bound = FP8_BOUND if self.bits == 8 else NVFP4_BOUND
            K.tensor_scale(inputs, bound, N.SCALAR_RCP, self.scratch, self.scale)
        if self.bits == 8:
            K.fp8_quantize(inputs, self.output, self.scale, N.SPEC_C)
        else:
            K.nvfp4_quantize(inputs, self.output, self.scales, self.blocked, self.scale, N.SPEC_C)
        return self
