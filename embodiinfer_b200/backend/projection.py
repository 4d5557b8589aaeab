"""Calibrated projections on the fused tensor-core Linear.

Drop-in for the reference's ``Projection`` / ``CalibratedProjectionBackend``
(embodiinfer/backend/torch/projection.py:15-254): weights are packed once, activations are encoded
at the fixed calibrated scale ``maximum / 448`` (FP8) or ``maximum / (448*6)`` (NVFP4) into
per-(shape, device, workspace) plans, and ``apply`` runs one launch that returns bf16 with the fp32
scales applied inside the kernel.  ``apply_gated`` is the fused gate/up + GELU + re-encode step the
reference needs two GEMMs and one elementwise kernel for (policies/pi05/inference/mlp.py:481-501).
"""

from __future__ import annotations

import math
from collections.abc import Callable

import torch

from .. import _native as N
from .. import kernels as K
from ..layers.plans import ActivationQuantizer, EncodedActivation, Precision, WorkspaceKey
from ..layers.registry import OperatorCapabilities
from ..weights import blocked_scales
from .quantization import blocked_scale_bytes


def gated_scale_layout(tokens: int, width: int) -> str:
    """Which of the two block-scale layouts an NVFP4 gate/up launch over ``tokens`` rows passes to ``b2_linear``.

    ``"paired"`` (64 gate rows + the 64 up rows of the same features per 128-row block) serves 64 + 64-column tiles:
    the single-CTA schedule, and on SM pairs the order that keeps the token rows on chip with two accumulators in
    tensor memory.  ``"bundle"`` (gate rows, then up rows) serves the 128 + 128-column tiles of SM pairs.  Measured
    on a B200 (microseconds, paired / bundle): 560 x 2 x 16384 x 2048 38.9 / 36.0; 8960 rows 352 / 322;
    640 x 2 x 4096 x 1024 11.0 / 12.1.  So: bundle for at least 2048 rows, and for prefill-sized launches (at least 512
    rows of width 2048 or more) whose last 256-row tile is mostly padding; paired otherwise."""
    if tokens >= 2048:
        return "bundle"
    padding = -(-tokens // 256) * 256 - tokens
    if tokens >= 512 and width >= 2048 and padding >= 128:
        return "bundle"
    return "paired"


class B200Projection:
    """One packed weight plus its execution-scoped activation encoders and output buffers."""

    def __init__(
        self,
        weight: torch.Tensor,
        maximum: float,
        precision: Precision,
        backend: ActivationQuantizer | None,
        workspace_key: Callable[[torch.device], WorkspaceKey] | None = None,
    ) -> None:
        if precision not in ("bf16", "fp8", "nvfp4"):
            raise ValueError("Projection precision must be bf16, fp8 or nvfp4")
        if weight.ndim != 2 or weight.dtype != torch.bfloat16:
            raise ValueError("Calibrated projections require a BF16 [output,input] weight")
        if not math.isfinite(maximum) or maximum <= 0:
            raise ValueError("Calibrated projection maximum must be finite and positive")
        if precision != "bf16" and (backend is None or weight.device.type != "cuda"):
            raise ValueError("Low precision projections require CUDA and an activation quantizer")
        if precision != "bf16" and torch.cuda.get_device_capability(weight.device) < (10, 0):
            raise ValueError(f"{precision} native GEMM requires SM (10, 0) or newer")
        self.precision, self.maximum, self.backend = precision, maximum, backend
        self.workspace_key = workspace_key or (lambda device: ("stream", torch.cuda.current_stream(device).cuda_stream))
        self.method = "bf16" if precision == "bf16" else f"calibrated_{precision}"
        self.output_dim, self.input_dim, self.device = weight.shape[0], weight.shape[1], weight.device
        self.plans: dict = {}
        self.outputs: dict = {}
        self.weight_scale_up: torch.Tensor | None = None   # set by `gated_pair`
        self.gated_flags = 0
        if precision == "bf16":
            self.bf16_weight = weight.detach()
        elif precision == "fp8":
            # projection.py:59-67: per-tensor amax/448, fp32 division, clamp, e4m3.
            values = weight.detach().contiguous().float()
            peak = values.abs().amax()
            self.weight_scale = torch.where(peak > 0, peak / 448.0, torch.ones_like(peak))
            self.weight_scale_1d = self.weight_scale.reshape(1)
            self.weight = (values / self.weight_scale).clamp(-448, 448).to(torch.float8_e4m3fn)
            self.weight_t = self.weight.t()
        else:
            # projection.py:69-74: the weight goes through the *activation* encoder in dynamic mode.
            source = weight.detach().contiguous()
            plan = backend.plan(source, 4).quantize(source)
            self.weight, self.weight_scale, self.weight_blocks = plan.output, plan.scale, plan.blocked
            self.weight_rowmajor_scales = plan.scales

    # -- activations ---------------------------------------------------------------------------
    def encode(self, inputs: torch.Tensor) -> EncodedActivation | None:
        """Encode activations at the calibrated scale; gate and up projections share one encoding."""
        if self.precision == "bf16":
            return None
        matrix = inputs.reshape(-1, inputs.shape[-1]).contiguous()
        key = (tuple(matrix.shape), matrix.device, self.workspace_key(matrix.device))
        if key not in self.plans:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm projection encoders before graph capture")
            bits = 8 if self.precision == "fp8" else 4
            self.plans[key] = self.backend.plan(matrix, bits, self.maximum / (448 * (6 if bits == 4 else 1)))
        return self.plans[key].quantize(matrix)

    def release_scope(self, scope: WorkspaceKey) -> None:
        """Drop the workspaces of one finished execution scope (projection.py:88-93).  The scope's launches have
        been waited for by then, so this is also where an expired bounded wait of one of them is reported."""
        if self.precision != "bf16":
            K.check_status(self.device)
        for key in tuple(self.plans):
            if key[-1] == scope:
                del self.plans[key]
        for key in tuple(self.outputs):
            if key[-1] == scope:
                del self.outputs[key]

    def _buffer(self, tag: str, shape: tuple[int, ...], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        key = (tag, shape, dtype, self.device, self.workspace_key(self.device))
        buffer = self.outputs.get(key)
        if buffer is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm projection outputs before graph capture")
            buffer = (torch.zeros if zero else torch.empty)(shape, device=self.device, dtype=dtype)
            self.outputs[key] = buffer
        return buffer

    def _scale_buffer(self, value: float) -> torch.Tensor:
        key = ("scale", value, self.device, self.workspace_key(self.device))
        buffer = self.outputs.get(key)
        if buffer is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm projection outputs before graph capture")
            buffer = torch.tensor(value, device=self.device, dtype=torch.float32)
            self.outputs[key] = buffer
        return buffer

    def _operands(self, encoded: EncodedActivation) -> dict:
        if self.precision == "fp8":
            return dict(kind=N.KIND_FP8, act=encoded.output, act_scale=encoded.scale, weight=self.weight,
                        weight_scale=self.weight_scale)
        return dict(kind=N.KIND_NVFP4, act=encoded.output, act_scales=encoded.blocked, act_scale=encoded.scale,
                    weight=self.weight, weight_scales=self.weight_blocks, weight_scale=self.weight_scale)

    def _check(self, inputs: torch.Tensor, encoded: EncodedActivation | None) -> None:
        if encoded is None or encoded.scale is None:
            raise ValueError("Low precision projections require encoded activations and a global scale")
        expected = self.input_dim if self.precision == "fp8" else self.input_dim // 2
        if inputs.device != self.device or inputs.dtype != torch.bfloat16 or encoded.output.shape[-1] != expected:
            raise ValueError("Projection input width, dtype or device changed")

    # -- GEMMs -------------------------------------------------------------------------------------
    def apply(
        self,
        inputs: torch.Tensor,
        encoded: EncodedActivation | None,
        *,
        bias: torch.Tensor | None = None,
        residual: torch.Tensor | None = None,
        rope: dict | None = None,
    ) -> torch.Tensor:
        """bf16 ``[..., N]``; optional bias and residual are added in the epilogue, each with its own
        bf16 rounding, exactly like separate ``output + bias`` / ``output + residual`` tensor adds.
        ``rope`` (FP8 packed QKV projections of at most 128 rows): the arguments of ``kernels.rope_split`` without
        ``qkv`` -- the launch writes rotated queries, keys and values to their buffers instead of returning the
        projection (``b2_linear_desc.rope``); the returned tensor is then not written."""
        shape = (*inputs.shape[:-1], self.output_dim)
        if self.precision == "bf16":
            if inputs.shape[-1] != self.input_dim or inputs.device != self.device or inputs.dtype != torch.bfloat16:
                raise ValueError("Projection input width, dtype or device changed")
            # Outside the quantised path: a plain library GEMM, as in the reference (projection.py:136-153).
            output = torch.nn.functional.linear(inputs.reshape(-1, self.input_dim), self.bf16_weight, bias)
            return (output if residual is None else output + residual.reshape(output.shape)).reshape(shape)
        self._check(inputs, encoded)
        rows = encoded.output.shape[0]
        output = self._buffer("linear", (rows, self.output_dim), torch.bfloat16)
        # More than one token tile: the library may cut a long K across SM pairs when few feature tiles exist
        # (e.g. the down projection of one observation: 560 x 2048 x 16384); it needs scratch for the partial sums.
        workspace = K.linear_workspace(self.device) if rows > 128 else None
        K.linear(
            epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=rows, features=self.output_dim, width=self.input_dim,
            out=output, bias=bias, residual=None if residual is None else residual.reshape(rows, self.output_dim),
            workspace=workspace, rope=rope, **self._operands(encoded),
        )
        return output.reshape(shape)

    def apply_gated(
        self,
        inputs: torch.Tensor,
        encoded: EncodedActivation | None,
        *,
        table: torch.Tensor,
        bits: int,
        scale: float | None = None,
        table_range: tuple[int, int] = (0, 0),
    ):
        """This weight is a packed ``[gate; up]`` (2F rows): one launch computes both projections,
        ``h = bf16(bf16(gelu(gate)) * up)`` and stores ``h`` as bf16 (``bits=16``), e4m3 (8) or
        NVFP4 (4) at the calibrated ``scale`` — the next projection's encoded input.

        Returns an object with ``output``, ``scale``, ``scales``, ``blocked`` like a quantisation plan.
        """
        if self.precision == "bf16":
            raise ValueError("apply_gated needs an fp8 or nvfp4 projection")
        if self.output_dim % 2:
            raise ValueError("a gated projection weight must hold gate rows followed by up rows")
        if bits not in (4, 8, 16) or (bits != 16 and (scale is None or not math.isfinite(scale) or scale <= 0)):
            raise ValueError("gated encoding requires bits 4/8/16 and a finite positive calibrated scale")
        self._check(inputs, encoded)
        rows, features = encoded.output.shape[0], self.output_dim // 2
        result = _GatedOutput()
        if bits == 16:
            result.output = self._buffer("gated16", (rows, features), torch.bfloat16)
            out_format = N.OUT_BF16
        else:
            result.scale = self._scale_buffer(float(scale))
            if bits == 8:
                result.output = self._buffer("gated8", (rows, features), torch.float8_e4m3fn)
                out_format = N.OUT_FP8
            else:
                result.output = self._buffer("gated4", (rows, features // 2), torch.uint8)
                result.scales = self._buffer("gated4_scales", (rows, features // 16), torch.float8_e4m3fn)
                result.blocked = self._buffer(
                    "gated4_blocked", (blocked_scale_bytes(rows, features),), torch.float8_e4m3fn, zero=True
                )
                out_format = N.OUT_NVFP4
        operands, flags = self._operands(encoded), self.gated_flags
        if (flags & N.LINEAR_PAIRED_GATE_UP_SCALES and getattr(self, "weight_blocks_bundle", None) is not None
                and gated_scale_layout(rows, self.input_dim) == "bundle"):
            operands["weight_scales"], flags = self.weight_blocks_bundle, flags & ~N.LINEAR_PAIRED_GATE_UP_SCALES
        K.linear(
            epilogue=N.EPI_GEGLU, out_format=out_format, tokens=rows, features=features, width=self.input_dim,
            out=result.output, gelu_table=table, out_scale=result.scale, out_scales=result.scales,
            out_blocked=result.blocked, weight_scale_up=self.weight_scale_up, gelu_range=table_range,
            flags=flags,
            **operands,
        )
        return result

    def apply_gelu(
        self,
        inputs: torch.Tensor,
        encoded: EncodedActivation | None,
        *,
        table: torch.Tensor,
        bias: torch.Tensor | None = None,
        bits: int = 16,
        scale: float | None = None,
        table_range: tuple[int, int] = (0, 0),
    ):
        """``h = gelu(x W^T + bias)`` in one launch (bias add and GELU with their bf16 roundings, GELU from the
        table), stored as bf16 (``bits=16``) or as e4m3 at the calibrated ``scale`` (``bits=8``): the fc1 of a
        SigLIP block together with the encoder of fc2's input (vision.py:441-576).  Returns an object with
        ``output`` and ``scale`` like a quantisation plan."""
        if self.precision == "bf16":
            raise ValueError("apply_gelu needs an fp8 or nvfp4 projection")
        if bits not in (8, 16) or (bits == 8 and (scale is None or not math.isfinite(scale) or scale <= 0)):
            raise ValueError("GELU encoding requires bits 8/16 and a finite positive calibrated scale")
        self._check(inputs, encoded)
        rows = encoded.output.shape[0]
        result = _GatedOutput()
        if bits == 16:
            result.output = self._buffer("gelu16", (rows, self.output_dim), torch.bfloat16)
        else:
            result.scale = self._scale_buffer(float(scale))
            result.output = self._buffer("gelu8", (rows, self.output_dim), torch.float8_e4m3fn)
        K.linear(
            epilogue=N.EPI_GELU, out_format=N.OUT_BF16 if bits == 16 else N.OUT_FP8, tokens=rows, features=self.output_dim,
            width=self.input_dim, out=result.output, bias=bias, gelu_table=table, out_scale=result.scale,
            gelu_range=table_range, **self._operands(encoded),
        )
        return result

    @classmethod
    def gated_pair(
        cls,
        gate_weight: torch.Tensor,
        up_weight: torch.Tensor,
        maximum: float,
        precision: Precision,
        backend: ActivationQuantizer | None,
        workspace_key: Callable[[torch.device], WorkspaceKey] | None = None,
    ) -> "B200Projection":
        """Pack separately quantised gate and up projections into one ``[gate; up]`` operand.

        Each half keeps the codes, block scales and per-tensor/global scale it would have as a
        projection of its own (projection.py:59-74), so ``apply_gated`` reproduces
        ``gate.apply`` / ``up.apply`` followed by the GELU epilogue; only the storage is shared.
        """
        if precision == "bf16":
            raise ValueError("gated_pair packs fp8 or nvfp4 projections")
        if gate_weight.shape != up_weight.shape:
            raise ValueError("gate and up projections must have the same shape")
        gate = cls(gate_weight, maximum, precision, backend, workspace_key)
        up = cls(up_weight, maximum, precision, backend, workspace_key)
        pair = cls.__new__(cls)
        pair.__dict__.update(gate.__dict__)
        pair.plans, pair.outputs = {}, {}
        pair.output_dim = 2 * gate.output_dim
        pair.weight = torch.cat((gate.weight.view(torch.uint8), up.weight.view(torch.uint8))).contiguous()
        pair.weight_scale, pair.weight_scale_up = gate.weight_scale, up.weight_scale
        if precision == "fp8":
            pair.weight = pair.weight.view(torch.float8_e4m3fn)
            pair.weight_scale_1d, pair.weight_t = gate.weight_scale.reshape(1), pair.weight.t()
        else:
            if gate.output_dim % 128:
                raise ValueError("NVFP4 gated pairs need an intermediate width divisible by 128")
            # Block scales in the paired row order the fused kernel reads fastest: 64 gate rows, then the
            # 64 up rows of the same features, and so on (B2_LINEAR_PAIRED_GATE_UP_SCALES).
            rows, blocks = gate.weight_rowmajor_scales.shape
            paired = torch.stack(
                (gate.weight_rowmajor_scales.view(torch.uint8).view(rows // 64, 64, blocks),
                 up.weight_rowmajor_scales.view(torch.uint8).view(rows // 64, 64, blocks)), dim=1,
            ).reshape(2 * rows, blocks)
            pair.weight_blocks = blocked_scales(paired)
            pair.gated_flags = N.LINEAR_PAIRED_GATE_UP_SCALES
            # ... and in bundle order (gate rows, then up rows) for the paired-SM schedule, whose 128 + 128 column
            # tiles read whole 128-row scale blocks
            pair.weight_blocks_bundle = blocked_scales(torch.cat(
                (gate.weight_rowmajor_scales.view(torch.uint8), up.weight_rowmajor_scales.view(torch.uint8))))
            pair.weight_rowmajor_scales = None
        return pair

    def refit_tensors(self, prefix: str = "") -> dict[str, torch.Tensor]:
        """The packed operands a weight refit has to refresh, by name: codes, block scales (every layout held) and
        per-tensor / global scales.  A refit copies new values INTO these tensors, so device pointers recorded in
        CUDA graphs and read by the launches stay valid (embodiinfer/engine/rollout/refit.py:122-137 runs its
        ``on_refit`` hook for the same reason)."""
        names = ("weight", "weight_scale", "weight_scale_up", "weight_blocks", "weight_blocks_bundle", "weight_rowmajor_scales",
                 "bf16_weight")
        found = {}
        for name in names:
            tensor = getattr(self, name, None)
            if isinstance(tensor, torch.Tensor):
                found[prefix + name] = tensor
        return found


class _GatedOutput:
    """Encoded activation produced by a fused epilogue (same attributes as a quantisation plan)."""

    output: torch.Tensor
    scale: torch.Tensor | None = None
    scales: torch.Tensor | None = None
    blocked: torch.Tensor | None = None
    dynamic = False


class B200ProjectionBackend:
    """Prepare bias-free bf16/FP8/NVFP4 projection weights without model knowledge."""

    capabilities = OperatorCapabilities(("cuda",), (torch.bfloat16,), "native_gemm_bf16_output", minimum_sm=(10, 0))

    def plan(
        self,
        weight: torch.Tensor,
        maximum: float,
        precision: Precision,
        quantizer: ActivationQuantizer | None,
        workspace_key: Callable[[torch.device], WorkspaceKey] | None = None,
    ) -> B200Projection:
        return B200Projection(weight, maximum, precision, quantizer, workspace_key)
