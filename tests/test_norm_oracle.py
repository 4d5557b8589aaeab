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


def test_layer_norm_restatement_tracks_torch_layer_norm():
    """The kernel-order LayerNorm stays within one bf16 unit in the last place of torch's fp32 layer_norm."""
    import torch
    rng = np.random.default_rng(13)
    for columns in (1152, 2048, 64):
        x = Q.f32_to_bf16(rng.standard_normal((9, columns)).astype(np.float32) * 2 + 0.3)
        update = Q.f32_to_bf16(rng.standard_normal((9, columns)).astype(np.float32))
        weight = Q.f32_to_bf16(rng.standard_normal(columns).astype(np.float32))
        bias = Q.f32_to_bf16(rng.standard_normal(columns).astype(np.float32))
        result = NO.layer_norm_quant(x, weight, bias, bits=16, update=update)
        residual = torch.from_numpy(Q.bf16_to_f32(result["residual"]))
        assert np.array_equal(result["residual"], Q.f32_to_bf16((Q.bf16_to_f32(x) + Q.bf16_to_f32(update)).astype(np.float32)))
        want = torch.nn.functional.layer_norm(residual, (columns,), torch.from_numpy(Q.bf16_to_f32(weight)),
                                              torch.from_numpy(Q.bf16_to_f32(bias)), 1e-6).numpy()
        got = Q.bf16_to_f32(result["output"])
        ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
        assert np.all(np.abs(got - want) <= np.maximum(ulp, 1e-2))
        assert np.allclose(result["mean"], residual.numpy().astype(np.float64).mean(axis=1), atol=1e-5)
    encoded = NO.layer_norm_quant(x, weight, bias, bits=8, scale_value=448.0 / 9.0)
    y = Q.bf16_to_f32(encoded["normalized"])
    assert np.array_equal(encoded["output"], Q.e4m3_encode_satfinite((y * np.float32(448.0 / 9.0)).astype(np.float32)))
    packed = NO.layer_norm_quant(x, weight, bias, bits=4, scale_value=9.0 / 2688.0)
    assert np.array_equal(packed["output"], Q.nvfp4_quantize_C(packed["normalized"], np.float32(9.0 / 2688.0))[0])


def test_layer_norm_sums_by_hand():
    """One thread's pair order and the two butterflies on a row that fits two warps."""
    row = (np.arange(1, 513, dtype=np.float32) / np.float32(7)).reshape(1, 512)
    total, squares = NO.layer_norm_sums(row, 5)
    lanes = row.reshape(64, 4, 2)
    per_thread = np.zeros(64, np.float32)
    for j in range(4):
        per_thread = (per_thread + (lanes[:, j, 0] + lanes[:, j, 1]).astype(np.float32)).astype(np.float32)
    warps = []
    for w in range(2):
        v = per_thread[32 * w:32 * w + 32].copy()
        for offset in (16, 8, 4, 2, 1):
            v = (v + v[np.arange(32) ^ offset]).astype(np.float32)
        warps.append(v[0])
    w0, w1, z = warps[0], warps[1], np.float32(0)
    expected = np.float32(np.float32(np.float32(w0 + z) + np.float32(z + z)) + np.float32(np.float32(w1 + z) + np.float32(z + z)))
    assert total[0] == expected and squares[0] > 0


def test_transposing_encoder_restatement():
    rng = np.random.default_rng(17)
    attended = Q.f32_to_bf16(rng.standard_normal((2, 3, 5, 16)).astype(np.float32))
    rows = NO.bhsd_quant(attended, 16)["output"]
    assert rows.shape == (10, 48)
    assert np.array_equal(rows[1 * 5 + 2, 16:32], attended[1, 1, 2])       # row b*S+s, columns h*D..h*D+D
    codes = NO.bhsd_quant(attended, 8, np.float32(100.0))["output"]
    assert np.array_equal(codes, Q.e4m3_encode_satfinite((Q.bf16_to_f32(rows) * np.float32(100.0)).astype(np.float32)))
    packed = NO.bhsd_quant(attended, 4, np.float32(0.003))
    assert np.array_equal(packed["output"], Q.nvfp4_quantize_C(rows, np.float32(0.003))[0])


def test_frames_oracle():
    from oracle import frames_oracle as FO
    frames = np.arange(2 * 4 * 6 * 3, dtype=np.uint8).reshape(2, 4, 6, 3)
    images = FO.normalize_frames(frames)
    assert images.shape == (2, 3, 4, 6) and images.dtype == np.float32
    assert images[0, 0, 0, 0] == np.float32(-1) and images[1, 2, 3, 5] == np.float32(np.float32(np.float32(143) / np.float32(255)) * np.float32(2)) - np.float32(1)
    patches = FO.frames_to_patches(frames, 2)
    assert patches.shape == (2 * 2 * 3, 12)
    # row (camera 1, patch row 1, patch column 2), column (channel 1, y 1, x 0) = pixel (y 3, x 4) of camera 1
    assert patches[1 * 6 + 1 * 3 + 2, 1 * 4 + 1 * 2 + 0] == Q.f32_to_bf16(images[1, 1, 3, 4].reshape(1))[0]
