"""A random-init policy with the shapes of the reference's pi0.5 stack, for rollout measurements.

Not a port of ``Pi05Policy``: no checkpoint, tokenizer or processor.  It strings together the layer
equations the reference runs (embodiinfer/policies/pi05/modeling_pi05.py:924-1168: pre-norm Gemma
blocks with a packed QKV projection, RoPE, grouped-query attention, gated GELU-tanh MLP; a SigLIP
vision tower; a 10-step flow-matching action expert that attends to the prefix keys/values and is
advanced by ``x += dt * v``, embodiinfer/models/schedulers/flow.py:21-23) at the widths the reference
guards for (operators.py:99-107, vision.py:276-601), with every q/k/v/o/gate/up/down/fc projection a
quantised ``FP8Linear`` / ``NVFP4Linear`` bundle dispatched through the registry to the sm_100a
kernels.  Norms, RoPE, softmax attention and the tiny action in/out projections are plain bf16 tensor
operations: they are not the quantised Linear this package is about.

Two MLP routes: the registry route (dynamic activation scales; gate_up Linear, GELU*up, down Linear as
separate steps, what ``QuantizedLinear.forward`` does in the reference) and, after
``calibrate_fused_mlp``, the calibrated plan route (``FusedMlpPlan``: encode, one fused gate_up + GELU*up
+ re-encode launch, down with the residual add in its epilogue), the counterpart of the reference's
``quantized_residual_mlp`` (policies/pi05/inference/operators.py:999-1037).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from . import kernels as K
from .backend.mlp import FusedGeluMlpPlan, FusedMlpPlan
from .backend.norm_quant import B200NormQuant
from .backend.projection import B200Projection
from .backend.quantization import B200Quantizer
from .bundles import pack_quantized_linears, quantize_linear
from .layers.linear import FP8Config, NVFP4Config, parse_quantization_config


@dataclass(frozen=True)
class TowerShape:
    width: int
    mlp: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int


GEMMA_2B = TowerShape(2048, 16384, 18, 8, 1, 256)
GEMMA_300M = TowerShape(1024, 4096, 18, 8, 1, 256)
SIGLIP_SO400M = TowerShape(1152, 4304, 27, 16, 16, 72)
IMAGE_SIZE, PATCH, CAMERAS, TEXT_TOKENS, VOCAB = 224, 14, 2, 48, 257152
ACTION_HORIZON, ACTION_DIM, DENOISE_STEPS = 10, 32, 10


def _random_linear(out_features: int, in_features: int, generator: torch.Generator, device, bias: bool = False) -> nn.Linear:
    layer = nn.Linear(in_features, out_features, bias=bias, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        layer.weight.copy_(0.02 * torch.randn((out_features, in_features), generator=generator, device=device))
        if bias:
            layer.bias.zero_()
    return layer


def _quantized(layers: tuple[nn.Linear, ...], config):
    members = tuple(quantize_linear(layer, config) for layer in layers)
    return members[0] if len(members) == 1 else pack_quantized_linears(members)


class _Shape:
    """Shape, dtype and device of an activation that only exists encoded."""

    def __init__(self, shape: tuple[int, ...], like: torch.Tensor) -> None:
        self.shape, self.device, self.dtype = torch.Size(shape), like.device, like.dtype


class FusedNorm:
    """RMSNorm + bf16 rounding + activation encoding at a calibrated projection's static scale in one launch
    (``NormQuantPlan.normalize``); one plan per activation shape and stream, created on first use."""

    def __init__(self, quantizer: B200Quantizer, projection: B200Projection) -> None:
        self.backend = B200NormQuant(quantizer)
        self.bits = 8 if projection.precision == "fp8" else 4
        self.scale = projection.maximum / (448 * (6 if self.bits == 4 else 1))
        self.plans: dict = {}

    def _plan(self, x: torch.Tensor, adaptive: bool):
        key = (tuple(x.shape), adaptive, torch.cuda.current_stream(x.device).cuda_stream)
        plan = self.plans.get(key)
        if plan is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm the fused norm before graph capture")
            plan = self.plans[key] = self.backend.plan(x, bits=self.bits, calibrated_scale=self.scale, adaptive=adaptive)
        return plan

    def __call__(self, x: torch.Tensor, weight: torch.Tensor):
        """``x``: contiguous bf16 [B, T, D]; ``weight``: fp32 [D] RMSNorm weight (the scale is 1 + weight)."""
        return self._plan(x, False).normalize(x, scale=weight)

    def modulated(self, x: torch.Tensor, modulation: torch.Tensor, pending=None):
        """Adaptive RMSNorm (``NormQuantPlan`` with ``adaptive=True``): ``modulation`` fp32 [B, 3D] = scale | shift |
        gate.  ``pending`` = (update, gate) of the sublayer before: the residual stream becomes
        ``x + update * gate`` in the same launch.  Returns (residual stream, encoded activation, this norm's gate)."""
        plan = self._plan(x, True)
        if pending is None:
            plan.normalize(x, modulation=modulation)
            return x, plan, plan.gate
        return plan.residual_normalize(x, pending[0].contiguous(), pending[1], modulation=modulation)


class FusedLayerNorm:
    """LayerNorm + bf16 rounding + e4m3 / NVFP4 encoding at a calibrated projection's static scale in one launch
    (``b2_layer_norm_quant``); one encoding workspace per activation shape and stream, created on first use."""

    def __init__(self, quantizer: B200Quantizer, projection: B200Projection) -> None:
        self.quantizer = quantizer
        self.bits = 8 if projection.precision == "fp8" else 4
        self.scale = projection.maximum / (448 * (6 if self.bits == 4 else 1))
        self.scale_value = 448.0 / projection.maximum if self.bits == 8 else self.scale
        self.plans: dict = {}

    def __call__(self, x: torch.Tensor, norm: nn.LayerNorm):
        rows = x.reshape(-1, x.shape[-1])
        key = (tuple(rows.shape), torch.cuda.current_stream(x.device).cuda_stream)
        plan = self.plans.get(key)
        if plan is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm the fused norm before graph capture")
            plan = self.plans[key] = self.quantizer.plan(rows, self.bits, self.scale)
        K.layer_norm_quant(rows, norm.weight, norm.bias, plan.output, bits=self.bits, scale_value=self.scale_value,
                           scales=plan.scales if self.bits == 4 else None, blocked=plan.blocked if self.bits == 4 else None)
        return plan


class FusedAttentionOutput:
    """Attention output [B, H, T, D] -> activations of the output projection [B*T, H*D], transposed and encoded at
    the projection's static scale in one launch (``b2_bhsd_quant``)."""

    def __init__(self, quantizer: B200Quantizer, projection: B200Projection) -> None:
        self.quantizer = quantizer
        self.bits = 8 if projection.precision == "fp8" else 4
        self.scale = projection.maximum / (448 * (6 if self.bits == 4 else 1))
        self.scale_value = 448.0 / projection.maximum if self.bits == 8 else self.scale
        self.plans: dict = {}

    def plan_for(self, attended: torch.Tensor):
        """The encoding workspace for an attention output shaped like ``attended`` [B, H, T, D] (only its shape and device
        are read)."""
        batch, heads, tokens, head_dim = attended.shape
        key = (batch * tokens, heads * head_dim, torch.cuda.current_stream(attended.device).cuda_stream)
        plan = self.plans.get(key)
        if plan is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm the attention-output encoder before graph capture")
            like = torch.empty((batch * tokens, heads * head_dim), device=attended.device, dtype=torch.bfloat16)
            plan = self.plans[key] = self.quantizer.plan(like, self.bits, self.scale)
        return plan

    def __call__(self, attended: torch.Tensor):
        plan = self.plan_for(attended)
        K.bhsd_quant(attended, plan.output, bits=self.bits, scale_value=self.scale_value,
                     scales=plan.scales if self.bits == 4 else None, blocked=plan.blocked if self.bits == 4 else None)
        return plan


class Projection(nn.Module):
    """One quantised Linear of the stack.  Registry route (the bundle, dynamic activation scale) until
    ``calibrate`` has seen its input range; afterwards the calibrated plan: static activation scale (no amax
    pass), bias and residual added in the GEMM's epilogue."""

    def __init__(self, layers: tuple[nn.Linear, ...], config) -> None:
        super().__init__()
        self.bundle = _quantized(layers, config)
        self.dense_weight = torch.cat([layer.weight.detach() for layer in layers]) if len(layers) > 1 else layers[0].weight.detach()
        self.dense_bias = None if layers[0].bias is None else torch.cat([layer.bias.detach() for layer in layers])
        self.method = "fp8" if isinstance(config, FP8Config) else "nvfp4" if isinstance(config, NVFP4Config) else None
        self.plan: B200Projection | None = None
        self.norm: FusedNorm | None = None
        self.layer_norm: FusedLayerNorm | None = None
        self.attention_output: FusedAttentionOutput | None = None
        self.maximum, self.recording = 0.0, False

    def attended(self, attended: torch.Tensor | None, residual: torch.Tensor, add_residual: bool = True, encoded=None) -> torch.Tensor:
        """``self(attended.transpose(1, 2).flatten(2), residual)`` for an attention output [B, H, T, D], the transpose
        and the activation encoding in one launch (calibrated plans only).  ``add_residual=False``: the projection
        alone, shaped like ``residual`` (the adaptive blocks add it through the next norm's gate).  ``encoded``: the
        attention kernel already wrote the encoded rows (``b2_attention_fp8``); ``attended`` is then not read."""
        rows = residual.reshape(-1, residual.shape[-1])
        if encoded is None:
            encoded = self.attention_output(attended)
        like = _Shape((rows.shape[0], self.plan.input_dim), rows)
        output = self.plan.apply(like, encoded, bias=self.dense_bias, residual=rows if add_residual else None)
        return output.reshape(residual.shape)

    def layer_normed(self, x: torch.Tensor, norm: nn.LayerNorm) -> torch.Tensor:
        """``self(norm(x))`` with the LayerNorm and the activation encoding in one launch (calibrated plans only)."""
        output = self.plan.apply(x.reshape(-1, x.shape[-1]), self.layer_norm(x.contiguous(), norm), bias=self.dense_bias)
        return output.reshape(*x.shape[:-1], output.shape[-1])

    def normed(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``self(RMSNorm(x))`` with the norm and the activation encoding in one launch (calibrated plans only)."""
        output = self.plan.apply(x.reshape(-1, x.shape[-1]), self.norm(x.contiguous(), weight), bias=self.dense_bias)
        return output.reshape(*x.shape[:-1], output.shape[-1])

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        if self.plan is not None:
            rows = x.reshape(-1, x.shape[-1])
            extra = None if residual is None else residual.reshape(-1, residual.shape[-1])
            output = self.plan.apply(rows, self.plan.encode(rows), bias=self.dense_bias, residual=extra)
            return output.reshape(*x.shape[:-1], output.shape[-1])
        if self.recording:
            self.maximum = max(self.maximum, float(x.abs().max()))
        output = self.bundle(x)
        return output if residual is None else output + residual

    def calibrate(self, quantizer: B200Quantizer, margin: float) -> None:
        if self.method is None or self.maximum <= 0.0:
            return
        self.plan = B200Projection(self.dense_weight.contiguous(), margin * self.maximum, self.method, quantizer)
        self.norm = FusedNorm(quantizer, self.plan)
        self.layer_norm = FusedLayerNorm(quantizer, self.plan)
        self.attention_output = FusedAttentionOutput(quantizer, self.plan)
        self.dense_bias = None if self.dense_bias is None else self.dense_bias.to(torch.bfloat16).contiguous()
        self.dense_weight = None


def _adarms_dense(width: int, generator, device) -> nn.Linear:
    """The modulation projection of one AdaRMS norm: small random weights, bias 0 | 0 | 1 (scale, shift, gate), so that a
    random-init stack keeps its sublayer outputs."""
    dense = nn.Linear(width, 3 * width, bias=True, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        dense.weight.copy_((0.02 * torch.randn((3 * width, width), generator=generator, device=device)).to(torch.bfloat16))
        dense.bias.zero_()
        dense.bias[2 * width:] = 1.0
    dense.requires_grad_(False)
    return dense


def _rms_norm(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Gemma RMSNorm, ``scale`` = 1 + weight (one fused kernel)."""
    return F.rms_norm(x, (x.shape[-1],), scale, 1e-6)


def _ada_rms_norm(x: torch.Tensor, modulation: torch.Tensor):
    """Adaptive RMSNorm as tensor operations (embodiinfer/policies/pi05/modeling_pi05.py:180-194): fp32 variance,
    ``normed * (1 + scale) + shift`` with fp32 scale | shift | gate [B, 3D]; returns (bf16 output, bf16 gate [B, 1, D])."""
    variance = x.float().square().mean(-1, keepdim=True)
    normed = x * torch.rsqrt(variance + 1e-6)
    scale, shift, gate = modulation.unsqueeze(1).chunk(3, dim=-1)
    return (normed * (1 + scale) + shift).to(x.dtype), gate.to(x.dtype)


def _gated_residual(x: torch.Tensor, pending) -> torch.Tensor:
    """``x + update * gate`` with both products rounded to bf16, as the fused producer does."""
    return x if pending is None else x + (pending[0] * pending[1])


def rope_tables(positions: torch.Tensor, head_dim: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(sine, cosine), fp32 [T, head_dim/2] for theta 1e4; computed once per forward, shared by all layers."""
    half = head_dim // 2
    frequency = torch.exp(-math.log(10000.0) * torch.arange(half, device=positions.device, dtype=torch.float32) / half)
    angles = positions.float()[:, None] * frequency[None, :]
    return angles.sin().contiguous(), angles.cos().contiguous()


def rope_reference(x: torch.Tensor, tables: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """x [..., T, D] bf16: the reference's rotation (backend/torch/rotary.py:24-27) as tensor operations:
    fp32 factors, separate multiplies and add/subtract, one rounding to bf16."""
    sine, cosine = tables
    first, second = x.chunk(2, dim=-1)
    return torch.cat((first * cosine - second * sine, second * cosine + first * sine), dim=-1).to(x.dtype)


class GemmaBlock(nn.Module):
    """Pre-norm block; ``prefix_kv`` lets the action expert attend to the prefix tower's keys/values."""

    def __init__(self, shape: TowerShape, attention_width: int, config, generator, device, adaptive: bool = False) -> None:
        super().__init__()
        self.shape = shape
        # adaptive (the action expert): both norms are AdaRMS norms whose scale | shift | gate come from the flow time
        # (a dense [width -> 3 width] per norm, evaluated once per schedule step outside the step's graph, as the
        # reference's runtime does: policies/pi05/inference/runtime.py:366-401), and each sublayer's output enters the
        # residual stream multiplied by its norm's gate
        self.adaptive = adaptive
        if adaptive:
            self.input_dense = _adarms_dense(shape.width, generator, device)
            self.post_dense = _adarms_dense(shape.width, generator, device)
        q_dim, kv_dim = shape.heads * shape.head_dim, shape.kv_heads * shape.head_dim
        make = lambda n, k: _random_linear(n, k, generator, device)
        self.qkv = Projection((make(q_dim, shape.width), make(kv_dim, shape.width), make(kv_dim, shape.width)), config)
        self.o_proj = Projection((make(shape.width, attention_width),), config)
        gate, up, down = make(shape.mlp, shape.width), make(shape.mlp, shape.width), make(shape.width, shape.mlp)
        self.gate_up = _quantized((gate, up), config)
        self.down = _quantized((down,), config)
        # bf16 originals, kept until `calibrate_fused_mlp` has built the calibrated plan (or dropped it)
        self.dense_mlp = (gate.weight.detach(), up.weight.detach(), down.weight.detach())
        self.method = "fp8" if isinstance(config, FP8Config) else "nvfp4" if isinstance(config, NVFP4Config) else None
        self.fused_mlp: FusedMlpPlan | None = None
        self.mlp_ranges = [0.0, 0.0]          # calibration: max |MLP input|, max |hidden|
        self.recording = False
        # scale = 1 + weight with zero-initialised weights (the random-init stacks use RMSNorm weights of 0)
        self.input_scale = nn.Parameter(torch.ones(shape.width, device=device, dtype=torch.bfloat16), requires_grad=False)
        self.post_scale = nn.Parameter(torch.ones(shape.width, device=device, dtype=torch.bfloat16), requires_grad=False)
        # the same norms as fp32 weights (scale - 1) for the fused norm + encoder launch of the calibrated plans
        self.input_weight = torch.zeros(shape.width, device=device)
        self.post_weight = torch.zeros(shape.width, device=device)
        self.mlp_norm: FusedNorm | None = None
        self.fused_norm = True
        self.native_attention = True        # b2_attention instead of torch's scaled_dot_product_attention (head dimension 256, one kv head)
        self.encode_in_attention = True     # the attention kernel writes the output projection's encoded input rows
        self.rope_in_projection = True      # adaptive blocks, FP8: the QKV projection's launch does the attention preparation

    def mlp(self, x: torch.Tensor) -> torch.Tensor:
        """x + down(gelu_tanh(gate(n)) * up(n)), n = RMSNorm(x)."""
        if self.fused_mlp is not None and self.mlp_norm is not None and self.fused_norm:
            rows = x.reshape(-1, x.shape[-1])
            return self.fused_mlp.project(rows, self.mlp_norm(x.contiguous(), self.post_weight), residual=rows).reshape(x.shape)
        normed = _rms_norm(x, self.post_scale)
        if self.fused_mlp is not None:
            rows = normed.reshape(-1, normed.shape[-1])
            return self.fused_mlp(rows, residual=x.reshape(rows.shape)).reshape(x.shape)
        gate, up = self.gate_up(normed).chunk(2, dim=-1)
        hidden = F.gelu(gate, approximate="tanh") * up
        if self.recording:
            self.mlp_ranges[0] = max(self.mlp_ranges[0], float(normed.abs().max()))
            self.mlp_ranges[1] = max(self.mlp_ranges[1], float(hidden.abs().max()))
        return x + self.down(hidden)

    def build_fused_mlp(self, quantizer: B200Quantizer, margin: float = 1.0) -> None:
        gate, up, down = self.dense_mlp
        self.fused_mlp = FusedMlpPlan(gate, up, down, gate_up_max=margin * self.mlp_ranges[0], down_max=margin * self.mlp_ranges[1],
                                      gate_up=self.method, down=self.method, quantizer=quantizer)
        self.mlp_norm = FusedNorm(quantizer, self.fused_mlp.gate_up) if self.method is not None else None
        self.dense_mlp = None

    def adaptive_mlp(self, x: torch.Tensor, attention_output: torch.Tensor, attention_gate: torch.Tensor, modulation: torch.Tensor):
        """The second half of an adaptive block: residual stream += attention output * gate, AdaRMS, gated MLP.  Returns
        (residual stream, (MLP output, its gate)): the MLP output joins the stream in the next norm's launch."""
        pending = (attention_output, attention_gate)
        if self.fused_mlp is not None and self.mlp_norm is not None and self.fused_norm:
            x, encoded, gate = self.mlp_norm.modulated(x.contiguous(), modulation, pending)
            rows = x.reshape(-1, x.shape[-1])
            return x, (self.fused_mlp.project(rows, encoded).reshape(x.shape), gate)
        x = _gated_residual(x, pending)
        normed, gate = _ada_rms_norm(x, modulation)
        if self.fused_mlp is not None:
            rows = normed.reshape(-1, normed.shape[-1])
            return x, (self.fused_mlp(rows).reshape(x.shape), gate)
        gate_half, up = self.gate_up(normed).chunk(2, dim=-1)
        hidden = F.gelu(gate_half, approximate="tanh") * up
        if self.recording:
            self.mlp_ranges[0] = max(self.mlp_ranges[0], float(normed.abs().max()))
            self.mlp_ranges[1] = max(self.mlp_ranges[1], float(hidden.abs().max()))
        return x, (self.down(hidden), gate)

    def forward(self, x, rope, kv_buffers=None, modulations=None, pending=None):
        """``kv_buffers`` (action expert): per-layer [B, 1, prefix + T, D] key/value buffers whose first
        ``prefix`` rows hold the prefix tower's keys/values; this block writes its own rows behind them.
        Adaptive blocks take ``modulations`` = (input norm's, post-attention norm's) fp32 [B, 3 width] and ``pending`` =
        (MLP output, gate) of the block before, and return (residual stream, own keys/values, pending)."""
        shape = self.shape
        batch, tokens, _ = x.shape
        attention_gate = None
        q = torch.empty((batch, shape.heads, tokens, shape.head_dim), device=x.device, dtype=x.dtype)
        if kv_buffers is None:
            k = torch.empty((batch, shape.kv_heads, tokens, shape.head_dim), device=x.device, dtype=x.dtype)
            v = torch.empty_like(k)
        else:
            k, v = kv_buffers
        preparation = dict(sine=rope[0], cosine=rope[1], q_out=q, k_out=k, v_out=v, batch=batch, tokens=tokens, heads=shape.heads,
                           kv_heads=shape.kv_heads, head_dim=shape.head_dim, kv_offset=k.shape[2] - tokens)
        qkv = None
        if self.adaptive:
            if self.qkv.norm is not None and self.fused_norm:
                x, encoded, attention_gate = self.qkv.norm.modulated(x.contiguous(), modulations[0], pending)
                # A packed FP8 QKV projection of a handful of rows: the attention preparation is the launch's epilogue
                # (b2_linear_desc.rope) -- measured faster than projection + b2_rope_split up to ~96 rows.
                if (self.rope_in_projection and self.qkv.plan.precision == "fp8" and self.qkv.dense_bias is None
                        and shape.head_dim == 256 and batch * tokens <= 96):
                    self.qkv.plan.apply(x.reshape(-1, x.shape[-1]), encoded, rope=preparation)
                else:
                    qkv = self.qkv.plan.apply(x.reshape(-1, x.shape[-1]), encoded, bias=self.qkv.dense_bias).reshape(batch, tokens, -1)
            else:
                x = _gated_residual(x, pending)
                normed, attention_gate = _ada_rms_norm(x, modulations[0])
                qkv = self.qkv(normed)
        elif self.qkv.norm is not None and self.fused_norm:
            qkv = self.qkv.normed(x, self.input_weight)
        else:
            qkv = self.qkv(_rms_norm(x, self.input_scale))
        q_dim = shape.heads * shape.head_dim
        if qkv is not None:
            # one launch: split, rotate q and k, [B, heads, T, D] queries, keys / values written into the buffers
            K.rope_split(qkv.reshape(batch * tokens, -1), **preparation)
        own_kv = (k, v)
        # b2_attention: one CTA per 128 query rows of a batch element; launches of few such tiles (a handful of observations'
        # ten-token chunks) cut the keys of a tile across a thread-block cluster instead of walking them serially
        # (measured, 8 heads x 10 queries over 570 keys: B = 1 / 8 / 32 / 64 take 7.2 / 7.8 / 11.4 / 14.5 us against
        # 11.3 / 20.7 / 33.1 / 63.0 for torch's kernel).
        native = self.native_attention and shape.head_dim == 256 and shape.kv_heads == 1
        output_encoder = self.o_proj.attention_output if self.fused_norm else None
        encoded = None
        # The attention kernel writes the encoded rows of the output projection itself (b2_attention_fp8 /
        # b2_attention_nvfp4): one launch less.  The NVFP4 encoding is some 150 instructions per 16 values on the four
        # epilogue warps of a CTA, which only pays on the latency chain of a small launch (B = 1 / 8: 7.27 -> 7.16 and
        # 9.45 -> 9.28 ms per chunk); the 560-token prefix (2.20 -> 2.40 ms per stack) and B = 64 keep the encoder launch.
        if native and output_encoder is not None and self.encode_in_attention and (output_encoder.bits == 8 or batch * tokens <= 128):
            encoded, attended = output_encoder.plan_for(q), None
            if output_encoder.bits == 8:
                K.attention(q, k, v, codes=encoded.output, multiplier=output_encoder.scale_value)
            else:
                K.attention(q, k, v, codes=encoded.output, blocked=encoded.blocked, scales=encoded.scales,
                            global_scale=output_encoder.scale_value)
        elif native:
            attended = K.attention(q, k, v)           # tcgen05 multi-query attention (b2_attention)
        else:
            attended = F.scaled_dot_product_attention(q, k, v, enable_gqa=shape.heads != shape.kv_heads)
        if self.adaptive:
            if self.o_proj.attention_output is not None and self.fused_norm:
                projected = self.o_proj.attended(attended, x, add_residual=False, encoded=encoded)
            else:
                projected = self.o_proj(attended.transpose(1, 2).reshape(batch, tokens, q_dim))
            x, pending = self.adaptive_mlp(x, projected, attention_gate, modulations[1])
            return x, own_kv, pending
        if self.o_proj.attention_output is not None and self.fused_norm:
            x = self.o_proj.attended(attended, x, encoded=encoded)
        else:
            x = self.o_proj(attended.transpose(1, 2).reshape(batch, tokens, q_dim), residual=x)
        return self.mlp(x), own_kv


class SiglipBlock(nn.Module):
    def __init__(self, shape: TowerShape, config, generator, device) -> None:
        super().__init__()
        self.shape = shape
        make = lambda n, k: _random_linear(n, k, generator, device, bias=True)
        width = shape.width
        self.qkv = Projection((make(3 * width, width),), config)
        self.out = Projection((make(width, width),), config)
        fc1, fc2 = make(shape.mlp, width), make(width, shape.mlp)
        self.fc1 = _quantized((fc1,), config)
        self.fc2 = _quantized((fc2,), config)
        self.dense_mlp = (fc1.weight.detach(), fc1.bias.detach(), fc2.weight.detach(), fc2.bias.detach())
        self.fused_mlp: FusedGeluMlpPlan | None = None
        self.mlp_ranges = [0.0, 0.0]
        self.recording = False
        self.norm1 = nn.LayerNorm(width, eps=1e-6, device=device, dtype=torch.bfloat16)
        self.norm2 = nn.LayerNorm(width, eps=1e-6, device=device, dtype=torch.bfloat16)
        self.mlp_norm: FusedLayerNorm | None = None
        self.fused_norm = True

    def forward(self, x):
        batch, tokens, width = x.shape
        heads, head_dim = self.shape.heads, self.shape.head_dim
        fused_norm = self.fused_norm and self.qkv.layer_norm is not None
        qkv = self.qkv.layer_normed(x, self.norm1) if fused_norm else self.qkv(self.norm1(x))
        q, k, v = qkv.view(batch, tokens, 3, heads, head_dim).permute(2, 0, 3, 1, 4)
        attended = F.scaled_dot_product_attention(q, k, v)
        if fused_norm:
            x = self.out.attended(attended, x)
        else:
            x = self.out(attended.transpose(1, 2).reshape(batch, tokens, width), residual=x)
        if self.fused_mlp is not None and self.mlp_norm is not None and self.fused_norm:
            rows = x.reshape(-1, width)
            return self.fused_mlp.project(rows, self.mlp_norm(x.contiguous(), self.norm2), residual=rows).reshape(x.shape)
        normed = self.norm2(x)
        if self.fused_mlp is not None:
            rows = normed.reshape(-1, width)
            return self.fused_mlp(rows, residual=x.reshape(rows.shape)).reshape(x.shape)
        hidden = F.gelu(self.fc1(normed), approximate="tanh")
        if self.recording:
            self.mlp_ranges[0] = max(self.mlp_ranges[0], float(normed.abs().max()))
            self.mlp_ranges[1] = max(self.mlp_ranges[1], float(hidden.abs().max()))
        return x + self.fc2(hidden)

    def build_fused_mlp(self, quantizer: B200Quantizer, margin: float = 1.0) -> None:
        fc1_weight, fc1_bias, fc2_weight, fc2_bias = self.dense_mlp
        self.fused_mlp = FusedGeluMlpPlan(fc1_weight, fc1_bias, fc2_weight, fc2_bias, fc1_max=margin * self.mlp_ranges[0],
                                          fc2_max=margin * self.mlp_ranges[1], quantizer=quantizer)
        self.mlp_norm = FusedLayerNorm(quantizer, self.fused_mlp.fc1)
        self.dense_mlp = None


def plan_tensors(module: nn.Module) -> dict[str, torch.Tensor]:
    """Every packed operand held by the calibrated plans below ``module`` (they are not module buffers), by a stable
    name: what a weight refit must refresh besides the state dict once ``calibrate_fused_mlp`` has run."""
    found: dict[str, torch.Tensor] = {}
    for name, child in module.named_modules():
        prefix = f"{name}." if name else ""
        plan = getattr(child, "plan", None)
        if isinstance(plan, B200Projection):
            found.update(plan.refit_tensors(prefix + "plan."))
        fused = getattr(child, "fused_mlp", None)
        if fused is not None:
            found.update(fused.refit_tensors(prefix + "fused_mlp."))
        bias = getattr(child, "dense_bias", None)
        if isinstance(bias, torch.Tensor) and plan is not None:
            found[prefix + "dense_bias"] = bias
    return found


class Pi05ShapedPolicy(nn.Module):
    """uint8 camera frames + text tokens -> [B, 10, 32] action chunk.

    ``layer_scale`` < 1 shortens every tower (tests use 2 layers); widths never change, so every
    quantised projection runs at its real shape.
    """

    def __init__(self, quantization="fp8", *, device="cuda", seed: int = 1005, layer_scale: float = 1.0,
                 vocabulary: int = VOCAB) -> None:
        super().__init__()
        device = torch.device(device)
        config = parse_quantization_config(quantization)
        # SigLIP's fc2 has K = 4304: its packed e2m1 rows (2152 bytes) are not a multiple of the 16 bytes a
        # TMA row pitch needs, so an NVFP4 policy keeps the vision tower in FP8 (as the reference's
        # nvfp4 presets do).
        vision_config = parse_quantization_config("fp8") if isinstance(config, NVFP4Config) else config
        generator = torch.Generator(device=device).manual_seed(seed)
        depth = lambda shape: max(1, round(shape.layers * layer_scale))
        self.vision = nn.ModuleList(SiglipBlock(SIGLIP_SO400M, vision_config, generator, device) for _ in range(depth(SIGLIP_SO400M)))
        self.prefix = nn.ModuleList(
            GemmaBlock(GEMMA_2B, GEMMA_2B.heads * GEMMA_2B.head_dim, config, generator, device) for _ in range(depth(GEMMA_2B))
        )
        self.expert = nn.ModuleList(
            GemmaBlock(GEMMA_300M, GEMMA_300M.heads * GEMMA_300M.head_dim, config, generator, device, adaptive=True)
            for _ in range(min(depth(GEMMA_300M), len(self.prefix)))
        )
        patches = (IMAGE_SIZE // PATCH) ** 2
        rand = lambda *shape: nn.Parameter(0.02 * torch.randn(shape, generator=generator, device=device).to(torch.bfloat16), requires_grad=False)
        self.patch_weight, self.patch_bias = rand(SIGLIP_SO400M.width, 3 * PATCH * PATCH), rand(SIGLIP_SO400M.width)
        self.position = rand(patches, SIGLIP_SO400M.width)
        self.vision_norm = nn.LayerNorm(SIGLIP_SO400M.width, eps=1e-6, device=device, dtype=torch.bfloat16)
        self.projector = Projection((_random_linear(GEMMA_2B.width, SIGLIP_SO400M.width, generator, device, bias=True),), vision_config)
        self.token_embedding = rand(vocabulary, GEMMA_2B.width)
        self.action_in, self.action_out = rand(GEMMA_300M.width, ACTION_DIM), rand(ACTION_DIM, GEMMA_300M.width)
        self.time_mlp = rand(GEMMA_300M.width, GEMMA_300M.width)
        self.final_dense = _adarms_dense(GEMMA_300M.width, generator, device)
        self.schedules: dict = {}
        self.quantizer = B200Quantizer() if isinstance(config, (FP8Config, NVFP4Config)) and device.type == "cuda" else None
        self.device_ = device
        self.noise_seed = seed

    # -- stages ----------------------------------------------------------------------------------
    def embed_images(self, images: torch.Tensor) -> torch.Tensor:
        """uint8 [B, cameras, H, W, 3] -> [B, cameras*256, 2048]; frames are scaled as (x/255)*2-1."""
        batch, cameras = images.shape[:2]
        grid = IMAGE_SIZE // PATCH
        frames = images.to(self.device_, non_blocking=True).reshape(batch * cameras, IMAGE_SIZE, IMAGE_SIZE, 3)
        # one launch: (x/255)*2-1 in fp32, bf16, and the (channel, y, x) patch gather of the patch embedding
        tiles = torch.empty((batch * cameras * grid * grid, 3 * PATCH * PATCH), device=self.device_, dtype=torch.bfloat16)
        K.frames_to_patches(frames.contiguous(), tiles, PATCH)
        tiles = tiles.view(batch * cameras, grid * grid, 3 * PATCH * PATCH)
        x = F.linear(tiles, self.patch_weight, self.patch_bias) + self.position
        for block in self.vision:
            x = block(x)
        return self.projector(self.vision_norm(x)).view(batch, cameras * grid * grid, GEMMA_2B.width)

    def encode_prefix(self, images: torch.Tensor, tokens: torch.Tensor):
        text = self.token_embedding[tokens.to(self.device_)] * math.sqrt(GEMMA_2B.width)
        x = torch.cat((self.embed_images(images), text.to(torch.bfloat16)), dim=1)
        rope = rope_tables(torch.arange(x.shape[1], device=self.device_), GEMMA_2B.head_dim)
        cache = []
        for block in self.prefix:
            x, kv = block(x, rope)
            cache.append(kv)
        return cache, x.shape[1]

    def modulation_schedule(self, batch: int):
        """Per Euler step, the fp32 [B, 3 width] scale | shift | gate of every AdaRMS norm of the expert (two per layer and
        the final one), from the step's flow time: sine/cosine features -> time MLP -> SiLU -> each norm's dense.  The
        times are fixed, so this is evaluated once per batch size and reused by every step's launches, like the
        reference's cached schedule (policies/pi05/inference/runtime.py:366-401)."""
        cached = self.schedules.get(batch)
        if cached is None:
            if torch.cuda.is_available() and self.device_.type == "cuda" and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm the modulation schedule before graph capture")
            half = GEMMA_300M.width // 2
            frequency = torch.exp(-math.log(10000.0) * torch.arange(half, device=self.device_) / half)
            denses = [dense for block in self.expert for dense in (block.input_dense, block.post_dense)] + [self.final_dense]
            rows = []
            for step in range(DENOISE_STEPS):
                angles = (1.0 - step / DENOISE_STEPS) * frequency
                features = torch.cat((angles.sin(), angles.cos())).to(torch.bfloat16)
                condition = F.silu(F.linear(features, self.time_mlp)).expand(batch, -1)
                rows.append(tuple(dense(condition).float().contiguous() for dense in denses))
            cached = self.schedules[batch] = tuple(rows)
        return cached

    def denoise(self, cache, prefix_length: int, noise: torch.Tensor) -> torch.Tensor:
        """``noise`` [B, 10, 32] fp32 ~ N(0, 1): ten Euler steps of the flow from t = 1 to t = 0.  The flow time reaches
        the expert only through its AdaRMS norms."""
        actions = noise
        rope = rope_tables(prefix_length + torch.arange(ACTION_HORIZON, device=self.device_), GEMMA_300M.head_dim)
        dt = -1.0 / DENOISE_STEPS
        schedule = self.modulation_schedule(noise.shape[0])
        # one key/value buffer per layer: the prefix rows are written once, the action rows every step
        buffers = []
        for keys, values in cache[: len(self.expert)]:
            pad = keys.new_zeros((*keys.shape[:2], ACTION_HORIZON, keys.shape[-1]))
            buffers.append((torch.cat((keys, pad), dim=2), torch.cat((values, pad), dim=2)))
        for step in range(DENOISE_STEPS):
            modulations = schedule[step]
            x = F.linear(actions.to(torch.bfloat16), self.action_in)
            pending = None
            for index, (block, kv) in enumerate(zip(self.expert, buffers)):
                x, _, pending = block(x, rope, kv_buffers=kv, modulations=modulations[2 * index: 2 * index + 2], pending=pending)
            final, _ = _ada_rms_norm(_gated_residual(x, pending), modulations[-1])
            velocity = F.linear(final, self.action_out).float()
            actions = actions + dt * velocity              # Euler step of the flow (flow.py:21-23)
        return actions

    def noise(self, batch: int) -> torch.Tensor:
        generator = torch.Generator(device=self.device_).manual_seed(self.noise_seed)
        return torch.randn((batch, ACTION_HORIZON, ACTION_DIM), device=self.device_, generator=generator)

    @torch.no_grad()
    def forward(self, observations: dict, noise: torch.Tensor | None = None) -> torch.Tensor:
        images, tokens = observations["images"], observations["tokens"]
        cache, prefix_length = self.encode_prefix(images, tokens)
        return self.denoise(cache, prefix_length, self.noise(images.shape[0]) if noise is None else noise)

    @torch.no_grad()
    def calibrate_fused_mlp(self, observations: dict, margin: float = 1.0) -> None:
        """Run ``observations`` through the registry route, record every MLP's input and hidden ranges, and
        switch the MLPs (Gemma: gated; SigLIP: bias + GELU, FP8) to the calibrated fused plans (three launches
        each, static scales) and the attention projections to calibrated plans (two launches each, bias and
        residual in the epilogue)."""
        blocks = [*self.vision, *self.prefix, *self.expert]
        projections = [module for module in self.modules() if isinstance(module, Projection)]
        for module in (*blocks, *projections):
            module.recording = True
        self.forward(observations)
        for block in blocks:
            block.recording = False
            block.build_fused_mlp(self.quantizer, margin)
        for projection in projections:
            projection.recording = False
            projection.calibrate(self.quantizer, margin)

    def refit_tensors(self) -> dict[str, torch.Tensor]:
        """Picked up by ``BroadcastWeightSync``: the calibrated plans' packed operands (see ``plan_tensors``)."""
        return plan_tensors(self)

    def flops_per_observation(self) -> float:
        """2*M*N*K over the quantised projections of one observation (attention and norms excluded)."""
        def block(shape, tokens, attention_width):
            q_dim, kv_dim = shape.heads * shape.head_dim, shape.kv_heads * shape.head_dim
            per_token = shape.width * (q_dim + 2 * kv_dim) + attention_width * shape.width + 3 * shape.width * shape.mlp
            return 2.0 * tokens * per_token
        vision_tokens = CAMERAS * (IMAGE_SIZE // PATCH) ** 2
        siglip = SIGLIP_SO400M
        vision = len(self.vision) * 2.0 * vision_tokens * (4 * siglip.width * siglip.width + 2 * siglip.width * siglip.mlp)
        vision += 2.0 * vision_tokens * siglip.width * GEMMA_2B.width
        prefix = len(self.prefix) * block(GEMMA_2B, vision_tokens + TEXT_TOKENS, GEMMA_2B.heads * GEMMA_2B.head_dim)
        expert = DENOISE_STEPS * len(self.expert) * block(GEMMA_300M, ACTION_HORIZON, GEMMA_300M.heads * GEMMA_300M.head_dim)
        return vision + prefix + expert


def synthetic_observations(count: int, seed: int = 1005, vocabulary: int = VOCAB) -> dict:
    """Seeded stand-ins with the reference's observation shapes: two 224x224 uint8 RGB cameras ~U[0,255]
    and 48 text tokens per observation (host tensors; the policy moves them to its device)."""
    generator = torch.Generator().manual_seed(seed)
    return {
        "images": torch.randint(0, 256, (count, CAMERAS, IMAGE_SIZE, IMAGE_SIZE, 3), dtype=torch.uint8, generator=generator),
        "tokens": torch.randint(0, vocabulary, (count, TEXT_TOKENS), generator=generator),
    }
