"""CPU oracle for the quantized-Linear hot path. TEST INFRASTRUCTURE ONLY.

This module restates, in numpy, the arithmetic of the reference's quantised
Linear path so that the CUDA kernels can be checked against it.  It is a
checker: the product (``embodiinfer_b200``) never imports it.  Only the tests,
the smoke entry and the CPU-baseline leg of the benchmark may call it.

Pinning: every function below is compared, bit for bit, against the reference's
own Python implementation imported on CPU (``tests/golden/make_golden.py``
generated the committed vectors; ``tests/test_oracle_golden.py`` replays them).
The GEMM *values* have no golden vector in the reference's own tests, so the
GEMM oracle is the composition "dequantise exactly, accumulate in float64,
apply the route's epilogue rounding"; that part is "parity unpinned" by the
reference's tests and pinned only by the reference functions it is composed of.

Two quantiser arithmetics exist in the reference, and both are restated:

* spec "T": the torch route
  (embodiinfer/backend/torch/fp8.py:66-73, embodiinfer/backend/torch/nvfp4.py:28-46)
* spec "C": the CUDA route
  (embodiinfer/backend/cuda/csrc/quantize.cu:38-104, embodiinfer/backend/torch/quantization.py:43-57)

ATen evaluates ``tensor / python_scalar`` as a true division on CPU but as a
multiplication by the rounded fp32 reciprocal on CUDA.  ``scalar_div`` selects
which one is restated: ``"div"`` (CPU ATen, what the golden vectors were made
with) or ``"rcp"`` (CUDA ATen, what the reference does on a GPU; also what
quantize.cu:54 does).

All bf16 tensors are carried as uint16 bit patterns, e4m3 as uint8 codes and
packed e2m1 as uint8 (low nibble = even column).
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
E4M3_MAX = F32(448.0)
E2M1_MAX = F32(6.0)
F32_TINY = np.finfo(np.float32).tiny

# --------------------------------------------------------------------------
# bf16 <-> fp32


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """Widen bf16 bit patterns (uint16) to float32 exactly."""
    bits = np.asarray(bits, dtype=np.uint16)
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round float32 to bf16 bit patterns, round-to-nearest-even (NaN kept quiet)."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    bits = values.view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    nan = np.isnan(values)
    out = rounded.astype(np.uint16)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def round_bf16(values: np.ndarray) -> np.ndarray:
    """float32 -> bf16 -> float32."""
    return bf16_to_f32(f32_to_bf16(values))


# --------------------------------------------------------------------------
# e4m3 (fn variant: no inf, 0x7f = NaN, max 448)


def _e4m3_positive_table() -> np.ndarray:
    codes = np.arange(0x7F, dtype=np.int64)  # 0x00 .. 0x7e
    exponent = codes >> 3
    mantissa = codes & 7
    normal = (1.0 + mantissa / 8.0) * np.exp2(exponent.astype(np.float64) - 7.0)
    subnormal = (mantissa / 8.0) * 2.0 ** -6
    return np.where(exponent == 0, subnormal, normal)


_E4M3_POS = _e4m3_positive_table()  # float64, exact
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0  # exact in float64


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn codes -> float32 (0x7f/0xff -> NaN)."""
    codes = np.asarray(codes, dtype=np.uint8)
    magnitude = codes & np.uint8(0x7F)
    table = np.concatenate([_E4M3_POS, [np.nan]]).astype(np.float32)
    values = table[magnitude]
    return np.where(codes & np.uint8(0x80), -values, values).astype(np.float32)


def e4m3_encode_satfinite(values: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn code, round-to-nearest-even, saturating to +-448.

    Restates ``__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)``
    (quantize.cu:63, 86) and, for inputs already clamped to +-448,
    ``tensor.to(torch.float8_e4m3fn)`` (fp8.py:72).
    """
    values = np.asarray(values, dtype=np.float32)
    magnitude = np.abs(values).astype(np.float64)
    index = np.searchsorted(_E4M3_MID, magnitude, side="left")  # midpoints strictly below
    # Exactly on a midpoint: pick the even code of the two neighbours.
    safe = np.minimum(index, len(_E4M3_MID) - 1)
    tie = (index < len(_E4M3_MID)) & (magnitude == _E4M3_MID[safe])
    index = np.where(tie & (index % 2 == 1), index + 1, index)
    index = np.minimum(index, 0x7E)
    code = index.astype(np.uint8)
    code = np.where(np.isnan(values), np.uint8(0x7F), code)
    sign = np.signbit(values).astype(np.uint8) << np.uint8(7)
    return (code | sign).astype(np.uint8)


# --------------------------------------------------------------------------
# e2m1

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_THRESHOLDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def e2m1_encode_rne(values: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 code with hardware semantics.

    Restates ``cvt.rn.satfinite.e2m1x2.f32`` (quantize.cu:14-20): ties to the
    even code, saturate at 6, the sign bit follows the input's sign bit (so a
    negative value that rounds to zero gives 0x8).  NaN gives 0x7 (positive max),
    which is what the PTX conversion returns for NaN inputs with satfinite.
    """
    values = np.asarray(values, dtype=np.float32)
    magnitude = np.abs(values)
    index = np.searchsorted(E2M1_THRESHOLDS, magnitude, side="left")
    safe = np.minimum(index, 6)
    tie = (index < 7) & (magnitude == E2M1_THRESHOLDS[safe])
    index = np.where(tie & (index % 2 == 1), index + 1, index)
    index = np.where(np.isnan(values), 7, index)
    sign = np.where(np.isnan(values), 0, np.signbit(values).astype(np.uint8) << np.uint8(3))
    return (index.astype(np.uint8) | sign.astype(np.uint8)).astype(np.uint8)


def e2m1_encode_bucketize(values: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit e2m1 code with the torch route's semantics (nvfp4.py:42-44).

    ``bucketize(abs(v), thresholds)`` sends ties toward zero and NaN to 7; the
    sign bit is ``v < 0`` (false for -0.0 and NaN).
    """
    values = np.asarray(values, dtype=np.float32)
    magnitude = np.searchsorted(E2M1_THRESHOLDS, np.abs(values), side="left").astype(np.uint8)
    sign = (values < 0).astype(np.uint8) << np.uint8(3)
    return (magnitude | sign).astype(np.uint8)


def e2m1_decode(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    values = E2M1_VALUES[codes & np.uint8(7)]
    return np.where(codes & np.uint8(8), -values, values).astype(np.float32)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[R, K] 4-bit codes -> [R, K/2] bytes, even column in the low nibble (nvfp4.py:45)."""
    return (codes[:, 0::2] | (codes[:, 1::2] << np.uint8(4))).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.asarray(packed, dtype=np.uint8)
    rows, half = packed.shape
    codes = np.empty((rows, half * 2), dtype=np.uint8)
    codes[:, 0::2] = packed & np.uint8(0x0F)
    codes[:, 1::2] = packed >> np.uint8(4)
    return codes


# --------------------------------------------------------------------------
# scalar helpers


def _scalar_divide(value: np.float32, divisor: float, scalar_div: str) -> np.float32:
    """``tensor / python_scalar`` as ATen evaluates it on CPU ("div") or CUDA ("rcp")."""
    if scalar_div == "div":
        return F32(F32(value) / F32(divisor))
    if scalar_div == "rcp":
        return F32(F32(value) * F32(F32(1.0) / F32(divisor)))
    raise ValueError("scalar_div must be 'div' or 'rcp'")


# --------------------------------------------------------------------------
# FP8 per-tensor quantisers


def fp8_scale_dynamic(x_bf16: np.ndarray, scalar_div: str = "div") -> np.float32:
    """Tensor amax -> scale = amax/448, 1.0 for an all-zero tensor.

    fp8.py:70-71, quantization.py:53-55, quantize.cu:47-55.
    """
    maximum = F32(np.max(np.abs(bf16_to_f32(x_bf16)))) if x_bf16.size else F32(0)
    if not maximum > 0:
        return F32(1.0)
    return _scalar_divide(maximum, 448.0, scalar_div)


def fp8_quantize_T(
    x_bf16: np.ndarray,
    scale: np.float32 | None = None,
    scalar_div: str = "div",
    divisor_bf16: bool = False,
):
    """Spec T (fp8.py:66-73): the quotient ``rows / scale`` is a bf16 tensor.

    ``rows`` is bf16 and ``scale`` a 0-dim fp32 tensor, so type promotion keeps
    bf16: the division is done in fp32 and the quotient is rounded to bf16,
    clamped to +-448 and converted to e4m3.  On CPU ATen treats the 0-dim
    divisor as a scalar and keeps it fp32 (``divisor_bf16=False``, what the
    golden vectors pin); ``divisor_bf16=True`` restates a kernel that first casts
    the 0-dim operand to the bf16 result type.
    Returns (codes uint8 [M,K], scale fp32) — the *unrounded* fp32 scale is what
    the GEMM later multiplies by.
    """
    if scale is None:
        scale = fp8_scale_dynamic(x_bf16, scalar_div)
    scale = F32(scale)
    divisor = round_bf16(np.array([scale], dtype=np.float32))[0] if divisor_bf16 else scale
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        quotient = round_bf16(bf16_to_f32(x_bf16) / divisor)
    quotient = np.clip(quotient, -E4M3_MAX, E4M3_MAX)
    return e4m3_encode_satfinite(quotient), scale


def fp8_quantize_C(x_bf16: np.ndarray, scale: np.float32 | None = None, scalar_div: str = "rcp"):
    """Spec C (quantize.cu:57-67, quantization.py:51-56): fp32 true division, satfinite."""
    if scale is None:
        scale = fp8_scale_dynamic(x_bf16, scalar_div)
    scale = F32(scale)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        quotient = (bf16_to_f32(x_bf16) / scale).astype(np.float32)
    return e4m3_encode_satfinite(quotient), scale


def fp8_quantize_weight_tensorwise(w_f32: np.ndarray, scalar_div: str = "div"):
    """fp8.py:32-40: fp32 weights, per-tensor scale, fp32 division, clamp, e4m3."""
    w = np.asarray(w_f32, dtype=np.float32)
    maximum = F32(np.max(np.abs(w)))
    scale = _scalar_divide(maximum, 448.0, scalar_div) if maximum > 0 else F32(1.0)
    quotient = np.clip((w / scale).astype(np.float32), -E4M3_MAX, E4M3_MAX)
    return e4m3_encode_satfinite(quotient), scale


# --------------------------------------------------------------------------
# NVFP4 quantisers


def swizzle_scales(scales: np.ndarray) -> np.ndarray:
    """Linear [R, Kb] e4m3 block scales -> the 128x4-tile layout, zero padded.

    nvfp4.py:14-25 and quantize.cu:97-101:
    offset = ((r/128)*ceil(Kb/4) + c/4)*512 + (r%32)*16 + ((r%128)/32)*4 + c%4.
    """
    scales = np.asarray(scales, dtype=np.uint8)
    rows, columns = scales.shape
    row_tiles = -(-rows // 128)
    column_tiles = -(-columns // 4)
    out = np.zeros(row_tiles * column_tiles * 512, dtype=np.uint8)
    r = np.arange(rows)[:, None]
    c = np.arange(columns)[None, :]
    offset = ((r // 128) * column_tiles + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    out[offset.ravel()] = scales.ravel()
    return out


def unswizzle_scales(blocked: np.ndarray, rows: int, columns: int) -> np.ndarray:
    column_tiles = -(-columns // 4)
    r = np.arange(rows)[:, None]
    c = np.arange(columns)[None, :]
    offset = ((r // 128) * column_tiles + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    return np.asarray(blocked, dtype=np.uint8)[offset]


def nvfp4_global_scale(x_f32: np.ndarray, spec: str, scalar_div: str) -> np.float32:
    """Global fp32 scale.  T: amax.clamp_min(tiny)/2688 (nvfp4.py:38).
    C: amax*(1/2688), 1.0 for an all-zero tensor (quantize.cu:54)."""
    maximum = F32(np.max(np.abs(x_f32))) if x_f32.size else F32(0)
    if spec == "T":
        return _scalar_divide(max(maximum, F32(F32_TINY)), 448.0 * 6.0, scalar_div)
    if not maximum > 0:
        return F32(1.0)
    return _scalar_divide(maximum, 448.0 * 6.0, "rcp")


def nvfp4_quantize_T(x: np.ndarray, scalar_div: str = "div", is_bf16: bool = True):
    """Spec T (nvfp4.py:28-46). ``x`` is bf16 bits [M,K] (or float32 when is_bf16=False).

    Returns (packed uint8 [M,K/2], block scales uint8 [M,K/16], global fp32).
    """
    values = bf16_to_f32(x) if is_bf16 else np.asarray(x, dtype=np.float32)
    rows, columns = values.shape
    if columns % 16:
        raise ValueError("NVFP4 quantization expects [M, K] with K divisible by 16")
    g = nvfp4_global_scale(values, "T", scalar_div)
    blocks = values.reshape(rows, columns // 16, 16)
    block_max = np.max(np.abs(blocks), axis=-1).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        if scalar_div == "div":
            sixth = (block_max / F32(6.0)).astype(np.float32)
        else:
            sixth = (block_max * F32(F32(1.0) / F32(6.0))).astype(np.float32)
        raw = (sixth / g).astype(np.float32)
        raw = np.clip(raw, F32(F32_TINY), E4M3_MAX)
        scale_codes = e4m3_encode_satfinite(raw)
        denominator = (g * e4m3_decode(scale_codes)).astype(np.float32)
        normalized = (blocks / denominator[..., None]).astype(np.float32)
        normalized = np.where(np.isnan(normalized), normalized, np.clip(normalized, -E2M1_MAX, E2M1_MAX))
    codes = e2m1_encode_bucketize(normalized.reshape(rows, columns))
    return pack_nibbles(codes), scale_codes, g


def nvfp4_quantize_C(x_bf16: np.ndarray, global_scale: np.float32 | None = None):
    """Spec C (quantize.cu:69-104).

    Returns (packed [M,K/2], linear scales [M,K/16], swizzled scales flat, global fp32).
    """
    values = bf16_to_f32(x_bf16)
    rows, columns = values.shape
    if columns % 16:
        raise ValueError("NVFP4 quantization expects K divisible by 16")
    g = nvfp4_global_scale(values, "C", "rcp") if global_scale is None else F32(global_scale)
    blocks = values.reshape(rows, columns // 16, 16)
    block_max = np.max(np.abs(blocks), axis=-1).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        raw = np.minimum(E4M3_MAX, (block_max / F32(F32(6.0) * g)).astype(np.float32))
        scale_codes = e4m3_encode_satfinite(raw)
        denominator = (g * e4m3_decode(scale_codes)).astype(np.float32)
        positive = denominator > 0
        safe = np.where(positive, denominator, F32(1.0))
        normalized = np.where(positive[..., None], (blocks / safe[..., None]).astype(np.float32), F32(0.0))
    codes = e2m1_encode_rne(normalized.reshape(rows, columns))
    return pack_nibbles(codes), scale_codes, swizzle_scales(scale_codes), g


def nvfp4_dequantize(packed: np.ndarray, scale_codes: np.ndarray, g: np.float32 | None) -> np.ndarray:
    """Packed codes + e4m3 block scales (+ global) -> float32 (nvfp4.py:49-66).
    With ``g=None`` only the block scales are applied."""
    codes = unpack_nibbles(packed)
    rows, columns = codes.shape
    values = e2m1_decode(codes).reshape(rows, columns // 16, 16)
    values = values * e4m3_decode(scale_codes)[..., None]
    if g is not None:
        values = values * F32(g)
    return values.reshape(rows, columns).astype(np.float32)


# --------------------------------------------------------------------------
# GELU(gate) * up epilogue (fusion.cu:5-10; activation.py:55-60)


def gelu_mul(gate_bf16: np.ndarray, up_bf16: np.ndarray, table_u16: np.ndarray) -> np.ndarray:
    """h = bf16(bf16(gelu(gate)) * up) with GELU read from a 65536-entry bf16 table.

    The table is indexed by the gate's bf16 bit pattern, exactly like the
    reference's kernels; it is built by the caller from the framework's GELU so
    that the two bf16 rounding points are the framework's.  Returns bf16 bits.
    """
    gelu = bf16_to_f32(np.asarray(table_u16, dtype=np.uint16)[np.asarray(gate_bf16, dtype=np.uint16)])
    return f32_to_bf16((gelu * bf16_to_f32(up_bf16)).astype(np.float32))


def gelu_tanh_table() -> np.ndarray:
    """A float64 restatement of F.gelu(x, approximate='tanh') over every bf16 input,
    rounded once to bf16.  Used only to cross-check the framework-built table."""
    with np.errstate(invalid="ignore", over="ignore"):
        x = bf16_to_f32(np.arange(65536, dtype=np.uint32).astype(np.uint16)).astype(np.float64)
        inner = 0.7978845608028654 * (x + 0.044715 * x * x * x)
        y = 0.5 * x * (1.0 + np.tanh(inner))
    return f32_to_bf16(y.astype(np.float32))


# --------------------------------------------------------------------------
# GEMM oracles (exact dequantised operands, float64 accumulation)


def _matmul64(a: np.ndarray, b_t: np.ndarray) -> np.ndarray:
    return a.astype(np.float64) @ b_t.astype(np.float64).T


def fp8_linear(a_codes, a_scale, w_codes, w_scale, bias_bf16=None) -> np.ndarray:
    """Y = bf16(acc * s_a * s_w) (+ bias as a separate bf16 add).  fp8.py:118-141,
    projection.py:155-163.  Returns bf16 bits [M, N]."""
    acc = _matmul64(e4m3_decode(a_codes), e4m3_decode(w_codes))
    y = f32_to_bf16((acc * float(F32(a_scale)) * float(F32(w_scale))).astype(np.float32))
    if bias_bf16 is not None:
        y = f32_to_bf16(bf16_to_f32(y) + bf16_to_f32(bias_bf16)[None, :])
    return y


def nvfp4_block_acc(a_packed, a_scales, w_packed, w_scales) -> np.ndarray:
    """float64 accumulation of block-scaled operands without global scales."""
    return _matmul64(nvfp4_dequantize(a_packed, a_scales, None), nvfp4_dequantize(w_packed, w_scales, None))


def nvfp4_linear_registry(a_packed, a_scales, a_g, w_packed, w_scales, w_g, bias_bf16=None) -> np.ndarray:
    """Registry route (nvfp4.py:109-123; quantize.cu:106-114):
    Y0 = bf16(acc); Y = bf16(Y0 * bf16(g_a*g_w)); then bias as a bf16 add."""
    y0 = round_bf16(nvfp4_block_acc(a_packed, a_scales, w_packed, w_scales).astype(np.float32))
    product = round_bf16(np.array([F32(a_g) * F32(w_g)], dtype=np.float32))[0]
    y = f32_to_bf16((y0 * product).astype(np.float32))
    if bias_bf16 is not None:
        y = f32_to_bf16(bf16_to_f32(y) + bf16_to_f32(bias_bf16)[None, :])
    return y


def nvfp4_linear_plan(a_packed, a_scales, a_g, w_packed, w_scales, w_g) -> np.ndarray:
    """Calibrated plan route (projection.py:224-234): fp32 global scales inside the GEMM."""
    acc = nvfp4_block_acc(a_packed, a_scales, w_packed, w_scales)
    return f32_to_bf16((acc * float(F32(a_g)) * float(F32(w_g))).astype(np.float32))


# --------------------------------------------------------------------------
# comparison helpers used by the parity tests


def rel_frobenius(got_bf16: np.ndarray, want_bf16: np.ndarray) -> float:
    got = bf16_to_f32(got_bf16).astype(np.float64)
    want = bf16_to_f32(want_bf16).astype(np.float64)
    denominator = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (denominator if denominator > 0 else 1.0))


def max_abs(got_bf16: np.ndarray, want_bf16: np.ndarray) -> float:
    got = bf16_to_f32(got_bf16).astype(np.float64)
    want = bf16_to_f32(want_bf16).astype(np.float64)
    return float(np.max(np.abs(got - want))) if got.size else 0.0
