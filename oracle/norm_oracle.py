"""CPU oracle for the RMSNorm / LayerNorm producers in front of the quantised projections.
TEST INFRASTRUCTURE ONLY: the product (``embodiinfer_b200``) never imports it.

Restates, in numpy fp32 (every product and sum rounded separately, as the reference's strict build with
``--fmad=false`` does), the arithmetic of

* embodiinfer/backend/cuda/csrc/norm_quant.cu:114-251 (256 strided lanes + halving tree),
  :254-369 and :381-514 (8 consecutive columns per lane + butterflies; widths 1024 and 2048),
  :5-89 (mean of squares supplied by the caller);
* embodiinfer/backend/torch/normalization.py:49-103 (the torch route: same affine arithmetic and rounding
  points on ``inputs.float().square().mean()`` and ``torch.rsqrt``).

Pinning: ``affine`` and ``residual_rows`` are compared bit for bit with the reference's ``TorchRMSNorm``
imported on CPU (``tests/golden/make_norm_golden.py`` made ``tests/golden/norm_golden.npz``; the golden
file carries torch's own ``rsqrt(mean + eps)`` so the oracle is fed the same factor).  The order of the
sums is the CUDA kernels' and has no CPU counterpart in the reference: that part is "parity unpinned" by
the reference's tests and restated from the kernel source only.

``rsqrtf`` is a hardware approximation (at most 2 ulp from the exact value per the CUDA math
documentation) whose bits a CPU cannot restate.  ``inverse_exact`` gives the correctly rounded value; GPU
tests read the kernel's own factor back, require it within 2 ulp of ``inverse_exact`` and then require
every output bit-exact given that factor.

bf16 tensors are carried as uint16 bit patterns.
"""

from __future__ import annotations

import numpy as np

from . import quant_oracle as Q

F32 = np.float32
EPS = F32(1.0e-6)


def residual_rows(inputs: np.ndarray, update: np.ndarray | None = None, update_gate: np.ndarray | None = None,
                  tokens: int = 1) -> np.ndarray:
    """bf16 [rows, columns] residual: ``bf16(input + bf16(update * gate[batch]))`` (norm_quant.cu:127-137,
    normalization.py:101).  Returns bf16 bit patterns."""
    values = Q.bf16_to_f32(inputs)
    if update is None:
        return np.asarray(inputs, dtype=np.uint16).copy()
    delta = Q.bf16_to_f32(update)
    if update_gate is not None:
        factor = np.repeat(Q.bf16_to_f32(update_gate), tokens, axis=0)
        delta = Q.round_bf16((delta * factor).astype(F32))
    return Q.f32_to_bf16((values + delta).astype(F32))


def _butterfly(values: np.ndarray, offsets) -> np.ndarray:
    """``v[i] = v[i] + v[i ^ offset]`` over the last axis for each offset in turn."""
    index = np.arange(values.shape[-1])
    for offset in offsets:
        values = (values + values[..., index ^ offset]).astype(F32)
    return values


def sum_squares_lanes8(rows: np.ndarray) -> np.ndarray:
    """Sum of squares per row in the order of norm_fp8_reduce_vec8 (norm_quant.cu:296-331): lane t adds
    columns 8t..8t+7 in turn, xor-butterfly over 32 lanes, xor-butterfly over 8 warp totals (absent warps
    count 0.0)."""
    rows = np.asarray(rows, dtype=F32)
    count, columns = rows.shape
    if columns % 256:
        raise ValueError("the 8-columns-per-lane order needs whole warps (columns % 256 == 0)")
    lanes = rows.reshape(count, columns // 8, 8)
    total = np.zeros(lanes.shape[:2], dtype=F32)
    for i in range(8):
        total = (total + (lanes[..., i] * lanes[..., i]).astype(F32)).astype(F32)
    warps = _butterfly(total.reshape(count, columns // 256, 32), (16, 8, 4, 2, 1))[..., 0]
    padded = np.zeros((count, 8), dtype=F32)
    padded[:, : warps.shape[1]] = warps
    return _butterfly(padded, (4, 2, 1))[:, 0]


def sum_squares_strided(rows: np.ndarray, lanes: int = 256) -> np.ndarray:
    """Sum of squares per row in the order of norm_fp8_reduce (norm_quant.cu:124-148): lane t adds columns
    t, t+256, ... in turn, then ``p[t] += p[t + stride]`` for stride 128 .. 1."""
    rows = np.asarray(rows, dtype=F32)
    count, columns = rows.shape
    padded = np.zeros((count, -(-columns // lanes) * lanes), dtype=F32)
    padded[:, :columns] = rows
    steps = padded.reshape(count, -1, lanes)
    partial = np.zeros((count, lanes), dtype=F32)
    for step in range(steps.shape[1]):
        valid = step * lanes + np.arange(lanes) < columns
        added = (partial + (steps[:, step] * steps[:, step]).astype(F32)).astype(F32)
        partial = np.where(valid, added, partial)
    stride = lanes // 2
    while stride:
        partial[:, :stride] = (partial[:, :stride] + partial[:, stride:2 * stride]).astype(F32)
        stride //= 2
    return partial[:, 0].copy()


def sum_squares(rows: np.ndarray) -> np.ndarray:
    """The order the reference launches for the width (norm_quant.cu:523-546)."""
    return sum_squares_lanes8(rows) if rows.shape[1] in (1024, 2048) else sum_squares_strided(rows)


def mean_term(total: np.ndarray, columns: int) -> np.ndarray:
    """``total * fp32(1/columns) + 1e-6`` in fp32 (norm_quant.cu:149): the argument of rsqrtf."""
    reciprocal = F32(F32(1.0) / F32(columns))
    return ((np.asarray(total, dtype=F32) * reciprocal).astype(F32) + EPS).astype(F32)


def inverse_exact(term: np.ndarray) -> np.ndarray:
    """Correctly rounded fp32 ``1/sqrt(term)``."""
    return (1.0 / np.sqrt(np.asarray(term, dtype=np.float64))).astype(F32)


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units of the last place between positive finite fp32 values."""
    return np.abs(np.asarray(a, dtype=F32).view(np.int32).astype(np.int64) - np.asarray(b, dtype=F32).view(np.int32).astype(np.int64))


def affine(residual: np.ndarray, inverse: np.ndarray, *, scale: np.ndarray | None = None,
           modulation: np.ndarray | None = None, tokens: int = 1) -> np.ndarray:
    """bf16 bits of ``(r * inv) * (1 + scale)`` or ``(r * inv) * (1 + m_scale) + m_shift``
    (norm_quant.cu:152-163, normalization.py:69-77).  ``modulation`` is fp32 [rows/tokens, 3*columns]."""
    values = Q.bf16_to_f32(residual)
    columns = values.shape[1]
    scaled = (values * np.asarray(inverse, dtype=F32).reshape(-1, 1)).astype(F32)
    if modulation is not None:
        modulation = np.repeat(np.asarray(modulation, dtype=F32), tokens, axis=0)
        multiplier = (F32(1.0) + modulation[:, :columns]).astype(F32)
        result = ((scaled * multiplier).astype(F32) + modulation[:, columns:2 * columns]).astype(F32)
    else:
        result = (scaled * (F32(1.0) + np.asarray(scale, dtype=F32)).astype(F32)).astype(F32)
    return Q.f32_to_bf16(result)


def modulation_gate(modulation: np.ndarray, columns: int) -> np.ndarray:
    """bf16 bits of the gate third of the modulation (norm_quant.cu:166-169)."""
    return Q.f32_to_bf16(np.asarray(modulation, dtype=F32)[:, 2 * columns:3 * columns])


def encode(normalized: np.ndarray, bits: int, global_scale, *, divide: bool = False) -> dict:
    """The encoder behind the norm: ``normalized`` is bf16 bits [rows, columns].

    bits 8: ``e4m3(y * fp32(1/g))`` (norm_quant.cu:150, 164-165) or, with ``divide`` (the given-mean kernel,
    norm_quant.cu:43-44), ``e4m3(y / g)``.  bits 4: NVFP4 spec C at ``g`` (norm_quant.cu:226-249)."""
    if bits == 16:
        return {"output": np.asarray(normalized, dtype=np.uint16)}
    g = F32(global_scale)
    if bits == 8:
        values = Q.bf16_to_f32(normalized)
        with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
            quotient = (values / g).astype(F32) if divide else (values * F32(F32(1.0) / g)).astype(F32)
        return {"output": Q.e4m3_encode_satfinite(quotient)}
    packed, scales, blocked, _ = Q.nvfp4_quantize_C(np.asarray(normalized, dtype=np.uint16), g)
    return {"output": packed, "scales": scales, "blocked": blocked}


def norm_quant(inputs: np.ndarray, *, bits: int, tokens: int = 1, scale=None, modulation=None, update=None,
               update_gate=None, mean=None, global_scale=None, inverse=None) -> dict:
    """The whole producer.  ``inverse`` overrides the factor (tests pass the device's own rsqrtf result);
    otherwise it is ``inverse_exact`` of the kernel-order mean (or of ``mean`` when given)."""
    residual = residual_rows(inputs, update, update_gate, tokens)
    values = Q.bf16_to_f32(residual)
    term = (np.asarray(mean, dtype=F32).reshape(-1) + EPS).astype(F32) if mean is not None \
        else mean_term(sum_squares(values), values.shape[1])
    factor = inverse_exact(term) if inverse is None else np.asarray(inverse, dtype=F32).reshape(-1)
    normalized = affine(residual, factor, scale=scale, modulation=modulation, tokens=tokens)
    result = encode(normalized, bits, global_scale, divide=mean is not None)
    result.update(residual=residual, normalized=normalized, term=term, inverse=factor)
    if modulation is not None:
        result["gate"] = modulation_gate(modulation, values.shape[1])
    return result


# --------------------------------------------------------------------------
# LayerNorm producer (SigLIP).  Restated from the kernel source only (norm_quant.cu:564-687, 797-931, built
# by the reference with --fmad=false): the reference has no CPU route with this arithmetic (its torch route
# calls F.layer_norm), so this part is "parity unpinned"; GPU tests feed the device's rsqrtf result back.


def layer_norm_sums(rows: np.ndarray, warps: int) -> tuple[np.ndarray, np.ndarray]:
    """Per-row sum and sum of squares in the kernels' order: thread t owns columns 8t..8t+7 and adds the pairs
    ``sum = sum + (x + y)``, ``sq = sq + (x*x + y*y)``; 32-lane xor-butterfly; xor-butterfly over the totals of
    ``warps`` warps (threads beyond the row contribute 0.0)."""
    rows = np.asarray(rows, dtype=F32)
    count, columns = rows.shape
    padded = np.zeros((count, warps * 256), dtype=F32)
    padded[:, :columns] = rows
    pairs = padded.reshape(count, warps * 32, 4, 2)
    total = np.zeros((count, warps * 32), dtype=F32)
    squares = np.zeros((count, warps * 32), dtype=F32)
    for j in range(4):
        x, y = pairs[:, :, j, 0], pairs[:, :, j, 1]
        total = (total + (x + y).astype(F32)).astype(F32)
        squares = (squares + ((x * x).astype(F32) + (y * y).astype(F32)).astype(F32)).astype(F32)
    results = []
    for values in (total, squares):
        per_warp = _butterfly(values.reshape(count, warps, 32), (16, 8, 4, 2, 1))[..., 0]
        eight = np.zeros((count, 8), dtype=F32)
        eight[:, :warps] = per_warp
        results.append(_butterfly(eight, (4, 2, 1))[:, 0])
    return results[0], results[1]


def layer_norm_quant(inputs: np.ndarray, weight: np.ndarray, bias: np.ndarray, *, bits: int, scale_value=1.0,
                     update: np.ndarray | None = None, deviation: np.ndarray | None = None) -> dict:
    """The whole LayerNorm producer on bf16 bit patterns.  ``deviation`` overrides ``1/sqrt(var + 1e-6)`` (tests
    pass the device's own rsqrtf result).  bits 8: ``e4m3(y * scale_value)``; bits 4: NVFP4 spec C at
    ``scale_value``; bits 16: y."""
    residual = residual_rows(inputs, update)
    values = Q.bf16_to_f32(residual)
    columns = values.shape[1]
    total, squares = layer_norm_sums(values, 5 if columns <= 1152 else 8)
    width = F32(columns)
    mean = (total / width).astype(F32)
    variance = np.maximum(F32(0.0), ((squares / width).astype(F32) - (mean * mean).astype(F32)).astype(F32))
    term = (variance + EPS).astype(F32)
    factor = inverse_exact(term) if deviation is None else np.asarray(deviation, dtype=F32).reshape(-1)
    centred = (values - mean[:, None]).astype(F32)
    scaled = ((centred * factor[:, None]).astype(F32) * Q.bf16_to_f32(weight)[None, :]).astype(F32)
    normalized = Q.f32_to_bf16((scaled + Q.bf16_to_f32(bias)[None, :]).astype(F32))
    if bits == 8:
        with np.errstate(over="ignore", invalid="ignore"):
            result = {"output": Q.e4m3_encode_satfinite((Q.bf16_to_f32(normalized) * F32(scale_value)).astype(F32))}
    else:
        result = encode(normalized, bits, scale_value)
    result.update(residual=residual, normalized=normalized, mean=mean, term=term, deviation=factor)
    return result


# --------------------------------------------------------------------------
# Attention output [B, H, S, D] -> encoded rows [B*S, H*D] (norm_quant.cu:689-795)


def bhsd_quant(attended: np.ndarray, bits: int, scale_value=1.0) -> dict:
    """``attended``: bf16 bits [B, H, S, D].  bits 8: ``e4m3(x * scale_value)`` (norm_quant.cu:705-712);
    bits 4: NVFP4 spec C at the global scale ``scale_value`` (norm_quant.cu:750-779); bits 16: the rows."""
    batch, heads, tokens, head_dim = attended.shape
    rows = np.ascontiguousarray(np.transpose(np.asarray(attended, dtype=np.uint16), (0, 2, 1, 3))).reshape(
        batch * tokens, heads * head_dim)
    if bits == 8:
        with np.errstate(over="ignore", invalid="ignore"):
            return {"output": Q.e4m3_encode_satfinite((Q.bf16_to_f32(rows) * F32(scale_value)).astype(F32))}
    return encode(rows, bits, scale_value)
