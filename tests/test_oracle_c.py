"""The plain-C restatement (oracle/quant_oracle.c, conversions by integer arithmetic on the float's bits)
against the numpy oracle (table search): two independent implementations of the CUDA-route arithmetic must
agree bit for bit, on every e4m3 / e2m1 rounding boundary and on the golden inputs' distributions."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import quant_oracle as O

ORACLE_DIR = Path(__file__).resolve().parents[1] / "oracle"


@pytest.fixture(scope="module")
def c_oracle():
    subprocess.run(["make", "-C", str(ORACLE_DIR)], check=True, capture_output=True)
    library = ctypes.CDLL(str(ORACLE_DIR / "_build" / "libquant_oracle_c.so"))
    library.oc_e4m3_encode.argtypes, library.oc_e4m3_encode.restype = [ctypes.c_float], ctypes.c_uint8
    library.oc_e2m1_encode.argtypes, library.oc_e2m1_encode.restype = [ctypes.c_float], ctypes.c_uint8
    library.oc_e4m3_decode.argtypes, library.oc_e4m3_decode.restype = [ctypes.c_uint8], ctypes.c_float
    pointer = ctypes.c_void_p
    library.oc_fp8_quantize.argtypes = [pointer, ctypes.c_int64, ctypes.c_float, pointer]
    library.oc_nvfp4_quantize.argtypes = [pointer, ctypes.c_int, ctypes.c_int, ctypes.c_float, pointer, pointer, pointer]
    return library


def boundary_values() -> np.ndarray:
    """Every midpoint between adjacent e4m3 and e2m1 magnitudes, its two float neighbours, the grid values
    themselves, saturation edges, zeros, infinities and NaN, both signs."""
    grid8 = np.array([v for v in O.e4m3_decode(np.arange(0x7f, dtype=np.uint8))], dtype=np.float64)
    grid4 = O.E2M1_VALUES.astype(np.float64)
    points = [grid8, grid4, (grid8[1:] + grid8[:-1]) / 2, (grid4[1:] + grid4[:-1]) / 2, np.array([448.0, 464.0, 480.0, 6.0, 7.0, 1e30, 1e-30])]
    values = np.concatenate(points).astype(np.float32)
    values = np.concatenate([values, np.nextafter(values, np.float32(np.inf)), np.nextafter(values, np.float32(-np.inf))])
    values = np.concatenate([values, -values, np.array([0.0, -0.0, np.inf, -np.inf, np.nan], dtype=np.float32)])
    return values.astype(np.float32)


def test_scalar_conversions_agree_on_every_rounding_boundary(c_oracle):
    values = boundary_values()
    random = np.random.default_rng(5).standard_normal(20000).astype(np.float32) * np.float32(40.0)
    for batch in (values, random):
        want8, want4 = O.e4m3_encode_satfinite(batch), O.e2m1_encode_rne(batch)
        got8 = np.array([c_oracle.oc_e4m3_encode(float(v)) for v in batch], dtype=np.uint8)
        got4 = np.array([c_oracle.oc_e2m1_encode(float(v)) for v in batch], dtype=np.uint8)
        assert np.array_equal(got8, want8), batch[got8 != want8][:8]
        assert np.array_equal(got4, want4), batch[got4 != want4][:8]
    codes = np.arange(256, dtype=np.uint8)
    decoded = np.array([c_oracle.oc_e4m3_decode(int(c)) for c in codes], dtype=np.float32)
    assert np.array_equal(decoded.view(np.uint32), O.e4m3_decode(codes).astype(np.float32).view(np.uint32)) or \
        np.array_equal(np.nan_to_num(decoded, nan=123.0), np.nan_to_num(O.e4m3_decode(codes).astype(np.float32), nan=123.0))


@pytest.mark.parametrize("rows,columns,outliers", [(37, 256, True), (130, 64, False), (3, 4304 // 16 * 16, True)])
def test_tensor_quantisers_agree_with_numpy_oracle(c_oracle, rows, columns, outliers):
    rng = np.random.default_rng(rows + columns)
    x = rng.standard_normal((rows, columns)).astype(np.float32)
    if outliers:
        x = np.where(rng.random((rows, columns)) < 0.01, x * 20, x)
    x[0, :16] = 0.0                                   # an all-zero block
    bf16 = O.f32_to_bf16(x.astype(np.float32))
    # FP8
    codes, scale = O.fp8_quantize_C(bf16)
    got = np.empty(bf16.size, dtype=np.uint8)
    c_oracle.oc_fp8_quantize(bf16.ctypes.data, bf16.size, float(scale), got.ctypes.data)
    assert np.array_equal(got.reshape(codes.shape), codes)
    # NVFP4
    packed, scales, blocked, g = O.nvfp4_quantize_C(bf16)
    got_packed, got_scales, got_blocked = np.empty_like(packed), np.empty_like(scales), np.zeros_like(blocked)
    c_oracle.oc_nvfp4_quantize(bf16.ctypes.data, rows, columns, float(g), got_packed.ctypes.data, got_scales.ctypes.data,
                               got_blocked.ctypes.data)
    assert np.array_equal(got_packed, packed) and np.array_equal(got_scales, scales) and np.array_equal(got_blocked, blocked)
