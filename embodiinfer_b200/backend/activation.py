"""GELU(gate) * up with calibrated re-encoding, as a stand-alone launch.

Drop-in for the reference's ``GeluMulFusion`` / ``FusionPlan``
(embodiinfer/backend/cuda/activation.py:13-168, csrc/fusion.cu).  The fused tensor-core Linear
(``B200Projection.apply_gated``) performs the same arithmetic in its epilogue; this class serves
callers that already hold bf16 gate/up matrices.
"""

from __future__ import annotations

from typing import Literal

import torch

from .. import _native as N
from .. import kernels as K
from ..layers.plans import ActivationQuantizer
from ..layers.registry import OperatorCapabilities


def gelu_table(device: torch.device, approximate: Literal["none", "tanh"] = "tanh") -> torch.Tensor:
    """bf16 GELU of every bf16 bit pattern, as uint16[65536] (activation.py:34-37).

    Built with the framework's own GELU on the target device so that the two bf16 rounding points
    of ``F.gelu(gate) * up`` are the framework's.
    """
    codes = torch.arange(65536, device=device, dtype=torch.int32).to(torch.uint16)
    return torch.nn.functional.gelu(codes.view(torch.bfloat16), approximate=approximate).view(torch.uint16)


class B200GeluMul:
    capabilities = OperatorCapabilities(
        ("cuda",),
        (torch.bfloat16,),
        "torch_gelu_product_bf16_rounding",
        rank=2,
        bits=(4, 8, 16),
        minimum_sm_by_bits=((4, (10, 0)),),
        minimum_sm=(10, 0),
    )

    def __init__(
        self, backend: ActivationQuantizer | None = None, *, approximate: Literal["none", "tanh"] = "none"
    ) -> None:
        if approximate not in ("none", "tanh"):
            raise ValueError("GELU approximation must be none or tanh")
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.backend, self.approximate = backend, approximate
        self.table = gelu_table(self.device, approximate)
        self.library = N.load()

    def plan(self, gate: torch.Tensor, bits: int, scale: float | None = None) -> "GeluMulPlan":
        return GeluMulPlan(self, gate, bits, scale)


class GeluMulPlan:
    """Fixed-shape output workspace; ``encode`` launches one kernel."""

    def __init__(self, backend: B200GeluMul, gate: torch.Tensor, bits: int, scale: float | None) -> None:
        if bits not in (4, 8, 16):
            raise ValueError("Expected bits in {4, 8, 16}")
        if gate.device != backend.device or gate.dtype != torch.bfloat16 or not gate.is_contiguous():
            raise ValueError("Fusion requires contiguous CUDA BF16 gate/up matrices")
        if gate.ndim != 2 or min(gate.shape) <= 0:
            raise ValueError("Fusion requires a matrix")
        self.backend, self.bits, self.shape = backend, bits, gate.shape
        self.quantized = None
        if bits == 16:
            self.output = torch.empty_like(gate)
            self.scale = self.scales = self.blocked = None
        else:
            if backend.backend is None:
                raise ValueError("Low precision GELU output requires an activation quantizer")
            if scale is None:
                raise ValueError("A single-pass fused quantizer requires a calibrated global scale")
            self.quantized = backend.backend.plan(gate, bits, scale)
            self.output = self.quantized.output
            self.scale, self.scales, self.blocked = self.quantized.scale, self.quantized.scales, self.quantized.blocked

    def _launch(self, gate: torch.Tensor, up: torch.Tensor | None, row_stride: int, packed: bool = False) -> None:
        rows, columns = self.shape
        # fusion.cu:109-135 picks the reciprocal-multiply encoder whenever the element count is a
        # multiple of eight and the true division otherwise (the packed entry always multiplies,
        # fusion.cu:167-200); follow it so the codes match.
        flags = 0 if packed or (rows * columns) % 8 == 0 else N.GEGLU_TRUE_DIV
        K.geglu(
            gate, up, self.output, bits=self.bits, table=self.backend.table, rows=rows, columns=columns,
            row_stride=row_stride, scale=self.scale, scales=self.scales if self.bits == 4 else None,
            blocked=self.blocked if self.bits == 4 else None, flags=flags,
        )

    def encode(self, gate: torch.Tensor, up: torch.Tensor) -> "GeluMulPlan":
        for tensor in (gate, up):
            if tensor.shape != self.shape or tensor.device != self.output.device:
                raise ValueError("Fusion input shape/device changed")
            if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
                raise ValueError("Fusion requires contiguous BF16 inputs")
        self._launch(gate, up, self.shape[1])
        return self

    def encode_packed(self, packed: torch.Tensor) -> "GeluMulPlan":
        """gate and up are the two halves of one contiguous [M, 2N] matrix (fusion.cu:167-200)."""
        rows, columns = self.shape
        if packed.shape != (rows, 2 * columns) or packed.dtype != torch.bfloat16 or not packed.is_contiguous():
            raise ValueError("Packed fusion input must be a contiguous BF16 [M, 2N] matrix")
        if self.bits == 4:
            raise ValueError("Packed GELU encoding supports 8- and 16-bit outputs")
        self._launch(packed, packed[:, columns:], 2 * columns, packed=True)
        return self
