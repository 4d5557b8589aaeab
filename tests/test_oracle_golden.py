"""The numpy oracle against vectors produced by the reference's own CPU code
(tests/golden/make_golden.py lists the reference functions).  Bit-exact."""

from __future__ import annotations

import hashlib

import numpy as np
import pytest

from oracle import quant_oracle as O
from tests.util import bits, gelu_table_cpu, make_input

SMALL = ("a", "b", "c", "d", "e")


@pytest.mark.parametrize("case", SMALL)
def test_fp8_activation_specs(golden, case):
    x = golden[f"{case}_x"]
    codes, scale = O.fp8_quantize_T(x, scalar_div="div")
    assert scale == golden[f"{case}_fp8T_scale"]
    assert np.array_equal(codes, golden[f"{case}_fp8T_codes"])
    codes, scale = O.fp8_quantize_C(x, scalar_div="div")
    assert scale == golden[f"{case}_fp8C_dyn_scale"]
    assert np.array_equal(codes, golden[f"{case}_fp8C_dyn_codes"])
    codes, _ = O.fp8_quantize_C(x, np.float32(0.0371))
    assert np.array_equal(codes, golden[f"{case}_fp8C_static_codes"])


@pytest.mark.parametrize("case", SMALL)
def test_nvfp4_torch_route(golden, case):
    x = golden[f"{case}_x"]
    packed, scales, g = O.nvfp4_quantize_T(x, "div")
    assert g == golden[f"{case}_nv4T_global"]
    assert np.array_equal(scales, golden[f"{case}_nv4T_scales"])
    assert np.array_equal(packed, golden[f"{case}_nv4T_packed"])
    assert np.array_equal(O.swizzle_scales(scales), golden[f"{case}_nv4T_blocked"])
    key = f"{case}_nv4T_dequant"
    if key in golden:
        assert np.array_equal(O.nvfp4_dequantize(packed, scales, g), golden[key])
    assert np.array_equal(O.unswizzle_scales(golden[f"{case}_nv4T_blocked"], *scales.shape), scales)


@pytest.mark.parametrize("case", SMALL)
def test_weight_quantisers(golden, case):
    w = golden[f"{case}_w"]
    codes, scale = O.fp8_quantize_weight_tensorwise(w, "div")
    assert scale == golden[f"{case}_wfp8_scale"]
    assert np.array_equal(codes, golden[f"{case}_wfp8_codes"])
    packed, scales, g = O.nvfp4_quantize_T(w, "div", is_bf16=False)
    assert g == golden[f"{case}_wnv4_global"]
    assert np.array_equal(scales, golden[f"{case}_wnv4_scales"])
    assert np.array_equal(packed, golden[f"{case}_wnv4_packed"])


@pytest.mark.parametrize("case", SMALL)
@pytest.mark.parametrize("approximate", ("tanh", "none"))
def test_gelu_product(golden, case, approximate):
    table = gelu_table_cpu(approximate)
    assert hashlib.sha256(table.tobytes()).hexdigest() == str(golden[f"gelu_table_{approximate}_sha256"])
    hidden = O.gelu_mul(golden[f"{case}_x"], golden[f"{case}_up"], table)
    want = golden[f"{case}_hidden_{approximate}"]
    # NaN payloads aside (none in these inputs) the two bf16 rounding points must agree bit for bit
    assert np.array_equal(hidden, want)


def test_benchmark_shapes_by_digest(golden):
    """Full-size configs: inputs regenerated from their seeds, outputs compared by SHA-256."""
    digests = dict(entry.split("=") for entry in golden["digests"].tolist())
    cases = {"cfg1_x": ((560, 2048), 1001), "cfg2_x": ((560, 2048), 1002), "cfg2_h": ((560, 16384), 1012)}

    def sha(array):
        return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()

    for name, (shape, seed) in cases.items():
        x = bits(make_input(shape, seed))
        assert sha(x) == digests[f"{name}_x"], "seeded input changed"
        codes, scale = O.fp8_quantize_T(x, scalar_div="div")
        assert sha(codes) == digests[f"{name}_fp8T_codes"] and sha(scale) == digests[f"{name}_fp8T_scale"]
        codes, scale = O.fp8_quantize_C(x, scalar_div="div")
        assert sha(codes) == digests[f"{name}_fp8C_dyn_codes"]
        packed, scales, g = O.nvfp4_quantize_T(x, "div")
        assert sha(packed) == digests[f"{name}_nv4T_packed"]
        assert sha(scales) == digests[f"{name}_nv4T_scales"]
        assert sha(g) == digests[f"{name}_nv4T_global"]
        assert sha(O.swizzle_scales(scales)) == digests[f"{name}_nv4T_blocked"]


def test_e4m3_and_e2m1_tables():
    """Round trip of every code and the documented tie rules."""
    codes = np.arange(256, dtype=np.uint8)
    finite = (codes & 0x7F) != 0x7F
    assert np.array_equal(O.e4m3_encode_satfinite(O.e4m3_decode(codes[finite])), codes[finite])
    assert O.e4m3_encode_satfinite(np.float32([1e9, -1e9, 448.0, 464.0])).tolist() == [0x7E, 0xFE, 0x7E, 0x7E]
    ties = np.float32([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.1])
    assert O.e2m1_decode(O.e2m1_encode_rne(ties)).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -0.0]
    assert O.e2m1_decode(O.e2m1_encode_bucketize(ties)).tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0]
    assert O.e2m1_encode_rne(np.float32([-0.1]))[0] == 8 and O.e2m1_encode_bucketize(np.float32([np.nan]))[0] == 7


def test_gemm_oracle_epilogues():
    """Route-specific rounding of the GEMM oracle on a case small enough to check by hand."""
    rng = np.random.default_rng(0)
    x = O.f32_to_bf16(rng.standard_normal((8, 64)).astype(np.float32))
    w = O.f32_to_bf16((rng.standard_normal((16, 64)) * 0.02).astype(np.float32))
    ap, asl, _, ag = O.nvfp4_quantize_C(x)
    wp, wsl, _, wg = O.nvfp4_quantize_C(w)
    plan = O.bf16_to_f32(O.nvfp4_linear_plan(ap, asl, ag, wp, wsl, wg))
    registry = O.bf16_to_f32(O.nvfp4_linear_registry(ap, asl, ag, wp, wsl, wg))
    dense = O.nvfp4_dequantize(ap, asl, ag).astype(np.float64) @ O.nvfp4_dequantize(wp, wsl, wg).astype(np.float64).T
    assert np.abs(plan - dense).max() <= np.abs(dense).max() * 2.0**-8
    assert np.abs(registry - dense).max() <= np.abs(dense).max() * 2.0**-6   # three bf16 roundings
