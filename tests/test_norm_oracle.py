"""The numpy norm oracle against vectors produced by the reference's TorchRMSNorm on CPU
(tests/golden/make_norm_golden.py), bit-exact, plus the properties of its two summation orders."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

from oracle import norm_oracle as NO
from oracle import quant_oracle as Q

CASES = ("plain", "wide", "residual", "adaptive", "adaptive_gated", "odd_width")


@pytest.fixture(scope="module")
def norm_golden():
    return dict(np.load(Path(__file__).parent / "golden" / "norm_golden.npz"))


@pytest.mark.parametrize("case", CASES)
def test_affine_and_residual_match_the_reference(norm_golden, case):
    g = norm_golden
    tokens = int(g[f"{case}_tokens"])
    residual = NO.residual_rows(g[f"{case}_inputs"], g.get(f"{case}_update"), g.get(f"{case}_update_gate"), tokens)
    assert np.array_equal(residual, g[f"{case}_residual"])
    normalized = NO.affine(residual, g[f"{case}_inverse"], scale=g.get(f"{case}_scale"),
                           modulation=g.get(f"{case}_modulation"), tokens=tokens)
    assert np.array_equal(normalized, g[f"{case}_normalized"])
    if f"{case}_gate" in g:
        assert np.array_equal(NO.modulation_gate(g[f"{case}_modulation"], residual.shape[1]), g[f"{case}_gate"])


@pytest.mark.parametrize("case", CASES)
def test_kernel_order_factor_is_close_to_the_reference_factor(norm_golden, case):
    """The CUDA kernels' summation orders give the reference's CPU factor to within fp32 summation noise."""
    g = norm_golden
    values = Q.bf16_to_f32(g[f"{case}_residual"])
    term = NO.mean_term(NO.sum_squares(values), values.shape[1])
    factor = NO.inverse_exact(term)
    assert np.all(NO.ulp_distance(factor, g[f"{case}_inverse"]) <= 16)


def test_summation_orders():
    rng = np.random.default_rng(7)
    rows = Q.round_bf16(rng.standard_normal((5, 2048)).astype(np.float32) * 3)
    exact = (rows.astype(np.float64) ** 2).sum(axis=1)
    for total in (NO.sum_squares_lanes8(rows), NO.sum_squares_strided(rows)):
        assert total.dtype == np.float32 and np.allclose(total, exact, rtol=2e-6)
    # a row whose squares are all 1.0 sums exactly in any order
    ones = np.ones((2, 1024), dtype=np.float32)
    assert np.array_equal(NO.sum_squares_lanes8(ones), np.full(2, 1024, np.float32))
    assert np.array_equal(NO.sum_squares_strided(ones[:, :960]), np.full(2, 960, np.float32))
    with pytest.raises(ValueError):
        NO.sum_squares_lanes8(np.zeros((1, 64), dtype=np.float32))


def test_strided_order_by_hand():
    """Three lanes' worth of a tiny row, written out: lane t adds t, t+4, ...; then the halving tree."""
    row = np.arange(1, 11, dtype=np.float32).reshape(1, 10)
    squares = (row[0] * row[0]).astype(np.float32)
    lanes = [np.float32(0)] * 4
    for column in range(10):
        lanes[column % 4] = np.float32(lanes[column % 4] + squares[column])
    expected = np.float32(np.float32(lanes[0] + lanes[2]) + np.float32(lanes[1] + lanes[3]))
    assert NO.sum_squares_strided(row, lanes=4)[0] == expected


def test_encode_and_whole_producer():
    rng = np.random.default_rng(11)
    inputs = Q.f32_to_bf16(rng.standard_normal((6, 1024)).astype(np.float32) * 2)
    scale = (rng.standard_normal(1024) * 0.1).astype(np.float32)
    out8 = NO.norm_quant(inputs, bits=8, tokens=3, scale=scale, global_scale=np.float32(0.02))
    y = Q.bf16_to_f32(out8["normalized"])
    reciprocal = np.float32(np.float32(1) / np.float32(0.02))
    assert np.array_equal(out8["output"], Q.e4m3_encode_satfinite((y * reciprocal).astype(np.float32)))
    given = NO.norm_quant(inputs, bits=8, tokens=3, scale=scale, global_scale=np.float32(0.02),
                          mean=(y.astype(np.float64) ** 2).mean(axis=1).astype(np.float32))
    assert np.array_equal(given["output"], Q.fp8_quantize_C(given["normalized"], np.float32(0.02))[0])
    out4 = NO.norm_quant(inputs, bits=4, tokens=3, scale=scale, global_scale=np.float32(0.004))
    packed, scales, blocked, _ = Q.nvfp4_quantize_C(out4["normalized"], np.float32(0.004))
    assert np.array_equal(out4["output"], packed) and np.array_equal(out4["scales"], scales)
    assert np.array_equal(out4["blocked"], blocked)
    assert np.all(NO.ulp_distance(out8["inverse"], NO.inverse_exact(out8["term"])) == 0)
    out16 = NO.norm_quant(inputs, bits=16, tokens=3, scale=scale)
    assert np.array_equal(out16["output"], out8["normalized"])
