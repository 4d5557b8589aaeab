"""Gated MLP as three launches: encode(x), [gate;up] GEMM + GELU + re-encode, down GEMM.

Replaces the chain of ``MlpPlan._project`` (embodiinfer/policies/pi05/inference/mlp.py:481-501):
encode once, ``gate.apply`` + ``up.apply`` (two library GEMMs writing bf16), ``fusion.encode``
(re-reads both), ``down.apply``.  Here gate and up are one fused tensor-core launch whose epilogue
emits the down projection's encoded input directly, so the [M, F] bf16 intermediates never reach HBM.
Arithmetic (rounding points, encoders, scales) is that of the separate steps.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence
from typing import Literal

import torch

from .. import kernels as K
from ..layers.plans import ActivationQuantizer, EncodedActivation, Precision, WorkspaceKey
from .activation import gelu_table
from .projection import B200Projection

_BITS = {"bf16": 16, "fp8": 8, "nvfp4": 4}


class FusedMlpPlan:
    """``down(gelu(gate(x)) * up(x))`` with calibrated activation ranges.

    ``gate_up_max`` / ``down_max`` are the calibrated absolute maxima of the MLP input and of the
    hidden activation (the reference's per-layer ``gate_up_max`` / ``down_max``); they fix the
    activation scales, so every launch is graph-capturable.
    """

    def __init__(
        self,
        gate_weight: torch.Tensor,
        up_weight: torch.Tensor,
        down_weight: torch.Tensor,
        *,
        gate_up_max: float,
        down_max: float,
        gate_up: Precision,
        down: Precision,
        quantizer: ActivationQuantizer,
        approximate: Literal["none", "tanh"] = "tanh",
        workspace_key: Callable[[torch.device], WorkspaceKey] | None = None,
        table: torch.Tensor | None = None,
        outliers: Sequence[int] | None = None,
    ) -> None:
        if gate_up == "bf16":
            raise ValueError("the fused MLP needs fp8 or nvfp4 gate/up projections")
        if gate_weight.shape != up_weight.shape or down_weight.shape != tuple(reversed(gate_weight.shape)):
            raise ValueError("Optimized MLP projection dimensions do not match")
        self.inter_size, self.hidden_size = gate_weight.shape
        # BF16 outlier channels (policies/pi05/inference/mlp.py:119-131): hidden channels whose range would dominate
        # their NVFP4 blocks are taken out of the quantised path (their gate/up rows and down columns are zeroed before
        # packing, so the kept channels no longer share block scales with them) and computed beside it in bf16.
        self.side_gate_up = self.side_down = None
        self._side_buffers: dict = {}
        self._workspace_key = workspace_key or (lambda device: ("stream", torch.cuda.current_stream(device).cuda_stream))
        if outliers is not None:
            if gate_up != "nvfp4":
                raise ValueError("BF16 outlier channels require NVFP4 gate/up projections")
            index = torch.tensor(tuple(outliers), dtype=torch.long, device=gate_weight.device)
            if index.numel() == 0 or int(index.max()) >= self.inter_size or int(index.min()) < 0:
                raise ValueError("Outlier channels exceed the MLP width")
            self.side_gate_up = torch.cat((gate_weight[index], up_weight[index]), dim=0).t().contiguous()
            self.side_down = down_weight[:, index].t().contiguous()
            gate_weight, up_weight, down_weight = (weight.clone() for weight in (gate_weight, up_weight, down_weight))
            gate_weight[index] = 0
            up_weight[index] = 0
            down_weight[:, index] = 0
        self.gate_up = B200Projection.gated_pair(gate_weight, up_weight, gate_up_max, gate_up, quantizer, workspace_key)
        self.down = B200Projection(down_weight, down_max, down, quantizer if down != "bf16" else None, workspace_key)
        self.table = gelu_table(gate_weight.device, approximate) if table is None else table
        self.approximate = approximate
        self.table_range = K.gelu_table_range(self.table)

    def encode(self, inputs: torch.Tensor) -> EncodedActivation:
        return self.gate_up.encode(inputs)

    def project(self, inputs: torch.Tensor, encoded: EncodedActivation, *, residual: torch.Tensor | None = None,
                normalized: torch.Tensor | None = None):
        """``encoded`` is ``inputs`` at the gate/up scale (shared by both halves, mlp.py:222).  With outlier channels,
        ``normalized`` is the bf16 MLP input (the norm's output) the side path multiplies; it defaults to ``inputs``,
        which is right unless the caller passes the residual stream there (the fused norm + encoder route)."""
        bits = _BITS[self.down.precision]
        scale = None if bits == 16 else self.down.maximum / (448 * (6 if bits == 4 else 1))
        hidden = self.gate_up.apply_gated(
            inputs, encoded, table=self.table, bits=bits, scale=scale, table_range=self.table_range
        )
        shape = (*inputs.shape[:-1], self.inter_size)
        if bits == 16:
            output = self.down.apply(hidden.output.reshape(shape), None)
        else:
            # The encoded hidden activation is complete; `apply` only reads shape/dtype/device of its first argument.
            output = self.down.apply(_ShapeOnly(shape, inputs), hidden, residual=residual)
        if self.side_down is not None:
            source = inputs if normalized is None else normalized
            if not isinstance(source, torch.Tensor):
                raise RuntimeError("BF16 outlier channels need the residual and norm of the fused NVFP4 input")
            self._add_outliers(source, output)
        return output

    def _add_outliers(self, normalized: torch.Tensor, output: torch.Tensor) -> None:
        """Accumulate the outlier channels' bf16 GELU(gate) * up and down projection into ``output``
        (mlp.py:242-260: two library GEMMs and one elementwise product, outside the quantised path)."""
        rows_in = normalized.reshape(-1, normalized.shape[-1])
        rows, width = rows_in.shape[0], self.side_down.shape[0]
        key = (rows, normalized.device, self._workspace_key(normalized.device))
        if key not in self._side_buffers:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm the BF16 outlier channels before graph capture")
            self._side_buffers[key] = (torch.empty((rows, 2 * width), device=normalized.device, dtype=torch.bfloat16),
                                       torch.empty((rows, width), device=normalized.device, dtype=torch.bfloat16))
        gate_up, hidden = self._side_buffers[key]
        torch.matmul(rows_in, self.side_gate_up, out=gate_up)
        torch.mul(torch.nn.functional.gelu(gate_up[:, :width], approximate=self.approximate), gate_up[:, width:], out=hidden)
        output.view(-1, output.shape[-1]).addmm_(hidden, self.side_down)

    def __call__(self, inputs: torch.Tensor, *, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.project(inputs, self.encode(inputs), residual=residual)

    def release_scope(self, scope: WorkspaceKey) -> None:
        self.gate_up.release_scope(scope)
        self.down.release_scope(scope)
        for key in tuple(self._side_buffers):
            if key[-1] == scope:
                del self._side_buffers[key]

    def refit_tensors(self, prefix: str = "") -> dict[str, torch.Tensor]:
        """Packed operands of both launches, for an in-place weight refit (see ``B200Projection.refit_tensors``)."""
        found = {**self.gate_up.refit_tensors(prefix + "gate_up."), **self.down.refit_tensors(prefix + "down.")}
        if self.side_down is not None:
            found[prefix + "side_gate_up"], found[prefix + "side_down"] = self.side_gate_up, self.side_down
        return found


class FusedGeluMlpPlan:
    """``fc2(gelu(fc1(x) + b1)) + b2`` with calibrated FP8 ranges in three launches: encode(x), fc1 + bias +
    GELU + e4m3 re-encode, fc2 + bias (+ residual).  The SigLIP block MLP of the reference's fast FP8 path
    (policies/pi05/inference/vision.py:441-576: fc1 GEMM + bias + tanh GELU + quant, fc2 GEMM + bias)."""

    def __init__(
        self,
        fc1_weight: torch.Tensor,
        fc1_bias: torch.Tensor | None,
        fc2_weight: torch.Tensor,
        fc2_bias: torch.Tensor | None,
        *,
        fc1_max: float,
        fc2_max: float,
        quantizer: ActivationQuantizer,
        approximate: Literal["none", "tanh"] = "tanh",
        workspace_key: Callable[[torch.device], WorkspaceKey] | None = None,
    ) -> None:
        if fc2_weight.shape != tuple(reversed(fc1_weight.shape)):
            raise ValueError("Optimized MLP projection dimensions do not match")
        self.inter_size = fc1_weight.shape[0]
        self.fc1 = B200Projection(fc1_weight, fc1_max, "fp8", quantizer, workspace_key)
        self.fc2 = B200Projection(fc2_weight, fc2_max, "fp8", quantizer, workspace_key)
        self.fc1_bias = None if fc1_bias is None else fc1_bias.detach().to(torch.bfloat16).contiguous()
        self.fc2_bias = None if fc2_bias is None else fc2_bias.detach().to(torch.bfloat16).contiguous()
        self.table = gelu_table(fc1_weight.device, approximate)
        self.table_range = K.gelu_table_range(self.table)

    def __call__(self, inputs: torch.Tensor, *, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.project(inputs, self.fc1.encode(inputs), residual=residual)

    def project(self, inputs: torch.Tensor, encoded: EncodedActivation, *, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``encoded`` is the MLP input at fc1's calibrated scale (e.g. written by the fused norm + encoder);
        ``inputs`` is only consulted for shape, dtype and device."""
        hidden = self.fc1.apply_gelu(inputs, encoded, table=self.table, bias=self.fc1_bias, bits=8,
                                     scale=self.fc2.maximum / 448, table_range=self.table_range)
        shape = (*inputs.shape[:-1], self.inter_size)
        return self.fc2.apply(_ShapeOnly(shape, inputs), hidden, bias=self.fc2_bias, residual=residual)

    def release_scope(self, scope: WorkspaceKey) -> None:
        self.fc1.release_scope(scope)
        self.fc2.release_scope(scope)

    def refit_tensors(self, prefix: str = "") -> dict[str, torch.Tensor]:
        found = {**self.fc1.refit_tensors(prefix + "fc1."), **self.fc2.refit_tensors(prefix + "fc2.")}
        for name in ("fc1_bias", "fc2_bias"):
            if getattr(self, name) is not None:
                found[prefix + name] = getattr(self, name)
        return found


class _ShapeOnly:
    """Stands in for the bf16 hidden activation that the fused epilogue never materialises."""

    def __init__(self, shape: tuple[int, ...], like: torch.Tensor) -> None:
        self.shape, self.device, self.dtype = torch.Size(shape), like.device, like.dtype
