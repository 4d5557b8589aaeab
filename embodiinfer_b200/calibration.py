"""Checkpoint-facing calibration for the fused MLP plans: the per-layer precision record, the schema-2
calibration loader and the SmoothQuant folding.

Mirrors, with the same names, validation and error messages,
``MlpLayerPrecision`` (embodiinfer/policies/pi05/inference/config.py:16-59), ``_apply_calibration``
(embodiinfer/policies/pi05/inference/presets.py:114-163) and ``smoothed_norm_scale`` / ``smoothed_adarms`` /
the weight folding of ``MlpPlan.__init__`` (embodiinfer/policies/pi05/inference/mlp.py:40-60, 108-131).  Host-side
tensor arithmetic only: nothing here launches a kernel of this package; ``fused_mlp_from_layer`` hands the
folded weights to ``FusedMlpPlan``.

The reference ships ranges for its own devices ("thor", "spark", "4090"); a B200 deployment passes its own
schema-2 file (or names one of those device keys explicitly).  The bf16 outlier side path, which the reference
ties to its Thor prefix tower (mlp.py:119-121), is available for any NVFP4 gate/up layer here.
"""

from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Literal, Mapping

import torch

Precision = Literal["bf16", "fp8", "nvfp4"]


@dataclass(frozen=True)
class MlpLayerPrecision:
    """Calibrated gate/up and down formats for one transformer MLP.

    ``smooth``: per-input-channel SmoothQuant scales (gate/up packed as ``W * s``, the preceding norm's output
    divided by ``s``).  ``outliers``: down-input channels a prefix NVFP4 MLP computes in bf16 beside the NVFP4 path.
    """

    gate_up: Precision = "bf16"
    down: Precision = "bf16"
    gate_up_max: float = 1.0
    down_max: float = 1.0
    smooth: tuple[float, ...] | None = None
    outliers: tuple[int, ...] | None = None

    def __post_init__(self) -> None:
        for precision in (self.gate_up, self.down):
            if precision not in ("bf16", "fp8", "nvfp4"):
                raise ValueError("MLP precision must be bf16, fp8 or nvfp4")
        if not (_positive_number(self.gate_up_max) and _positive_number(self.down_max)):
            raise ValueError("Activation maxima must be finite and positive")
        if self.smooth is not None:
            scales = tuple(self.smooth)
            object.__setattr__(self, "smooth", scales)
            if len(scales) == 0 or not all(_positive_number(value) for value in scales):
                raise ValueError("SmoothQuant scales must be finite and positive")
            if self.gate_up == "bf16":
                raise ValueError("SmoothQuant scales apply to quantized gate/up projections")
        if self.outliers is not None:
            channels = tuple(self.outliers)
            object.__setattr__(self, "outliers", channels)
            valid = len(channels) > 0 and all(type(index) is int and index >= 0 for index in channels)
            if not valid or len(set(channels)) != len(channels):
                raise ValueError("Outlier channels must be distinct non-negative integers")
            if self.gate_up != "nvfp4":
                raise ValueError("BF16 outlier channels require NVFP4 gate/up projections")


def _positive_number(value) -> bool:
    """A Python int or float (not bool, not a numpy scalar: the reference checks the exact type), finite, > 0."""
    return type(value) in (int, float) and math.isfinite(value) and value > 0


@dataclass(frozen=True)
class Calibration:
    """Per-tower MLP ranges of one checkpoint (``prefix_layers`` / ``action_layers`` of the reference's
    ``Pi05OptimizationConfig``); a tower run in bf16 keeps ``None``."""

    prefix_layers: tuple[MlpLayerPrecision, ...] | None
    action_layers: tuple[MlpLayerPrecision, ...] | None
    checkpoint_sha256: str


def load_calibration(
    source: str | Path | Mapping,
    *,
    hardware: str,
    formats: Mapping[str, Precision],
    numerics: str = "openpi_rlinf",
    activation: str = "gelu_pytorch_exact",
    layers_per_tower: int = 18,
) -> Calibration:
    """Read a schema-2 calibration (a path, or the parsed document) and select the ranges of ``hardware`` for
    the towers in ``formats`` (``{"prefix": "nvfp4", "action": "fp8"}``).  Same checks, in the same order and
    with the same messages, as the reference's ``_apply_calibration``."""
    data = json.loads(Path(source).read_text()) if isinstance(source, (str, Path)) else source
    if not isinstance(data, Mapping) or (
        type(data.get("schema_version")) is not int
        or data.get("schema_version") != 2
        or data.get("numerics") != numerics
        or data.get("activation") != activation
    ):
        raise ValueError("Calibration must identify schema 2 and the matching numerical contract")
    devices = data.get("devices")
    ranges = devices.get(hardware) if isinstance(devices, Mapping) else None
    if not isinstance(ranges, Mapping):
        raise ValueError(f"Calibration has no ranges for {hardware}")
    layers: dict[str, tuple[MlpLayerPrecision, ...]] = {}
    for tower, precision in formats.items():
        if precision == "bf16":
            continue
        choices = ranges.get(tower)
        rows = choices.get(precision) if isinstance(choices, Mapping) else None
        if not isinstance(rows, list) or len(rows) != layers_per_tower:
            raise ValueError(f"Calibration requires {layers_per_tower} {tower} MLP layer ranges for {precision}")
        values = tuple(MlpLayerPrecision(**row) for row in rows)
        if not any(precision in (layer.gate_up, layer.down) for layer in values) or any(
            value not in ("bf16", precision) for layer in values for value in (layer.gate_up, layer.down)
        ):
            raise ValueError(f"Calibration {tower} formats must select {precision} with optional BF16 protection")
        layers[f"{tower}_layers"] = values
    if data.get("checkpoint_sha256") is None:
        raise ValueError("Calibration requires a checkpoint SHA256")
    return Calibration(layers.get("prefix_layers"), layers.get("action_layers"), data["checkpoint_sha256"])


def smoothed_norm_scale(weight: torch.Tensor, smooth: torch.Tensor) -> torch.Tensor:
    """fp32 RMSNorm scale (applied as ``1 + w``) whose output is divided by the SmoothQuant scales."""
    return ((1.0 + weight.float()) * (1.0 / smooth) - 1.0).contiguous()


def smoothed_adarms(weight: torch.Tensor, bias: torch.Tensor, smooth: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """AdaRMS ``[scale, shift, gate]`` projection (weight [3D, C], bias [3D]) whose normalised output is divided
    by the scales: ``1 + scale' = (1 + scale) / s`` and ``shift' = shift / s``; the residual-gate rows stay.
    Arithmetic in fp32 in the reference's order (rows times ``1/s``; scale bias ``b/s + (1/s - 1)``), results in
    the parameters' dtypes."""
    reciprocal = 1.0 / smooth
    width = reciprocal.numel()
    rows = weight.float().clone().view(3, width, -1)
    offsets = bias.float().clone().view(3, width)
    rows[0] *= reciprocal[:, None]
    rows[1] *= reciprocal[:, None]
    offsets[0] = offsets[0] * reciprocal + (reciprocal - 1.0)
    offsets[1] *= reciprocal
    return rows.view(3 * width, -1).to(weight.dtype), offsets.view(3 * width).to(bias.dtype)


def smoothed_projection_weights(gate_weight: torch.Tensor, up_weight: torch.Tensor, layer: MlpLayerPrecision):
    """Gate and up weights with the layer's SmoothQuant scales folded into their input channels
    (``W * s`` in fp32, rounded back to the weight dtype); unchanged without scales."""
    if layer.smooth is None:
        return gate_weight, up_weight
    smooth = torch.tensor(layer.smooth, dtype=torch.float32, device=gate_weight.device)
    if smooth.numel() != gate_weight.shape[1]:
        raise ValueError("SmoothQuant scales must match the MLP input width")
    return (gate_weight.float() * smooth).to(gate_weight.dtype), (up_weight.float() * smooth).to(up_weight.dtype)


def fused_mlp_from_layer(gate_weight: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor,
                         layer: MlpLayerPrecision, quantizer, **options):
    """``FusedMlpPlan`` for one calibrated layer record: validates the checkpoint layout like the reference's
    ``MlpPlan``, folds SmoothQuant scales into gate/up and passes the layer's formats and ranges on.  The caller
    divides the preceding norm by the same scales (``smoothed_norm_scale`` / ``smoothed_adarms``)."""
    from .backend.mlp import FusedMlpPlan
    weights = (gate_weight, up_weight, down_weight)
    if any(weight.dtype != torch.bfloat16 for weight in weights):
        raise ValueError("Optimized Pi05 MLPs require bias-free BF16 projection weights")
    if gate_weight.shape != up_weight.shape or down_weight.shape != tuple(reversed(gate_weight.shape)):
        raise ValueError("Optimized Pi05 MLP projection dimensions do not match")
    gate_weight, up_weight = smoothed_projection_weights(gate_weight.detach(), up_weight.detach(), layer)
    if layer.outliers is not None and max(layer.outliers) >= gate_weight.shape[0]:
        raise ValueError("Outlier channels exceed the MLP width")
    return FusedMlpPlan(gate_weight, up_weight, down_weight.detach(), gate_up_max=layer.gate_up_max, down_max=layer.down_max,
                        gate_up=layer.gate_up, down=layer.down, quantizer=quantizer, outliers=layer.outliers, **options)


# ---- deployment recipes -------------------------------------------------------------------------------------
# Counterpart of ``resolve_preset`` (embodiinfer/policies/pi05/inference/presets.py:27-112): one name selects the
# formats of the prefix and action towers' MLPs, the calibration supplies the per-layer ranges, and the recipe names
# the operator back ends a policy should ask the registries for.  The reference has launch profiles for "thor",
# "spark", "orin" and "4090"; this package adds the one for "b200" and keeps the reference's preset names, checks
# and messages.

_FORMATS = ("bf16", "fp8", "nvfp4")
_OPTIMIZED = {"bf16": ("bf16", "bf16"),
              **{f"{prefix}-{action}": (prefix, action) for prefix in _FORMATS for action in _FORMATS if (prefix, action) != ("bf16", "bf16")}}
DEVICES = ("b200",)


@dataclass(frozen=True)
class Recipe:
    """What a preset resolves to: tower formats, per-layer calibrated ranges (``None`` for a bf16 tower) and the back-end
    names to request from ``quantization_backends`` / ``projection_backends`` / ``gelu_mul_backends`` /
    ``norm_quant_backends`` (the names ``embodiinfer_b200.integration.register_into_reference`` registers)."""

    hardware: str
    prefix: Precision = "bf16"
    action: Precision = "bf16"
    prefix_layers: tuple[MlpLayerPrecision, ...] | None = None
    action_layers: tuple[MlpLayerPrecision, ...] | None = None
    checkpoint_sha256: str | None = None
    fused_mlp: bool = False
    numerics: str = "openpi_rlinf"
    activation: str = "gelu_pytorch_exact"
    operators: Mapping[str, str] | None = None

    @property
    def has_quantized_mlp(self) -> bool:
        return self.prefix != "bf16" or self.action != "bf16"


def resolve_preset(device: str, preset: str, *, calibration: str | Path | Mapping | None) -> Recipe:
    """Resolve one complete recipe; format names are ordered prefix then action (``"nvfp4-fp8"``)."""
    if device not in DEVICES:
        raise ValueError(f"Unknown Pi05 device {device!r}; choose from {DEVICES}")
    if preset == "strict":
        if calibration is not None:
            raise ValueError("The strict BF16 preset does not use calibration")
        return Recipe(hardware=device)
    if preset in ("w4a16", "w8a8-w4a16"):
        raise ValueError("Integer MLP presets require Orin and an offline calibrated weight manifest")
    if preset not in _OPTIMIZED:
        raise ValueError("Pi05 preset must be strict, bf16, w4a16, w8a8-w4a16 or a prefix-action format pair")
    prefix, action = _OPTIMIZED[preset]
    operators = {"quantization": "b200", "projection": "b200", "gelu_mul": "b200", "norm_quant": "b200", "attention_projection": "b200"}
    recipe = Recipe(hardware=device, prefix=prefix, action=action, fused_mlp=True, operators=operators)
    if not recipe.has_quantized_mlp:
        return recipe
    if calibration is None:
        raise ValueError(f"Calibration has no ranges for {device}")      # the reference falls back to its bundled file, which has no B200 entry
    found = load_calibration(calibration, hardware=device, formats={"prefix": prefix, "action": action},
                             numerics=recipe.numerics, activation=recipe.activation)
    return Recipe(hardware=device, prefix=prefix, action=action, prefix_layers=found.prefix_layers, action_layers=found.action_layers,
                  checkpoint_sha256=found.checkpoint_sha256, fused_mlp=True, operators=operators)
