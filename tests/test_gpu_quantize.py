"""Activation quantisers on the GPU, through the C ABI, against the oracle.  Bit-exact."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from embodiinfer_b200 import _native as N
from embodiinfer_b200 import kernels as K
from embodiinfer_b200.backend.quantization import blocked_scale_bytes
from oracle import quant_oracle as O
from tests.util import bits, make_input, u8

pytestmark = pytest.mark.gpu

SHAPES = [(37, 64), (560, 2048), (130, 256), (16, 64), (3, 16), (1, 16), (129, 192), (17, 4304 - 4304 % 16)]


def run_scale(x, bound, flags):
    scratch = K.new_scale_scratch(x.device)
    scale = torch.full((), -1.0, device=x.device)
    K.tensor_scale(x, bound, flags, scratch, scale)
    torch.cuda.synchronize()
    assert scratch.tolist() == [0, 0], "the scale kernel must leave its scratch zeroed"
    return scale


@pytest.mark.parametrize("shape", SHAPES)
def test_fp8_all_modes(device, shape):
    x = make_input(shape, 11 + shape[0])
    xb, xd = bits(x), x.to(device)
    for flags, mode in ((0, "div"), (N.SCALAR_RCP, "rcp")):
        assert np.float32(run_scale(xd, 448.0, flags).item()) == O.fp8_scale_dynamic(xb, mode)
    scale_value = O.fp8_scale_dynamic(xb, "rcp")
    scale = torch.tensor(float(scale_value), device=device)
    out = torch.empty(shape, device=device, dtype=torch.uint8)
    for flags, want in (
        (N.SPEC_T, O.fp8_quantize_T(xb, scale_value)[0]),
        (N.SPEC_T | N.DIVISOR_BF16, O.fp8_quantize_T(xb, scale_value, divisor_bf16=True)[0]),
        (N.SPEC_C, O.fp8_quantize_C(xb, scale_value)[0]),
    ):
        out.fill_(0xAA)
        K.fp8_quantize(xd, out, scale, flags)
        assert np.array_equal(u8(out), want), f"flags={flags}"


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] % 16 == 0])
def test_nvfp4_all_modes(device, shape):
    rows, columns = shape
    x = make_input(shape, 23 + rows)
    xb, xd = bits(x), x.to(device)
    packed = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8)
    blocked = torch.empty(blocked_scale_bytes(rows, columns), device=device, dtype=torch.uint8)
    cases = (
        ("C", N.SCALAR_RCP, N.SPEC_C, O.nvfp4_quantize_C(xb)),
        ("T/div", N.CLAMP_TINY, N.SPEC_T, O.nvfp4_quantize_T(xb, "div")),
        ("T/rcp", N.CLAMP_TINY | N.SCALAR_RCP, N.SPEC_T | N.SCALAR_RCP, O.nvfp4_quantize_T(xb, "rcp")),
    )
    for name, scale_flags, flags, want in cases:
        g = run_scale(xd, 448.0 * 6.0, scale_flags)
        assert np.float32(g.item()) == want[-1], name
        blocked.zero_()
        K.nvfp4_quantize(xd, packed, linear, blocked, g, flags)
        assert np.array_equal(u8(packed), want[0]), name
        assert np.array_equal(u8(linear), want[1]), name
        assert np.array_equal(u8(blocked), O.swizzle_scales(want[1])), name
    # optional outputs may be omitted
    K.nvfp4_quantize(xd, packed, None, None, g, N.SPEC_T | N.SCALAR_RCP)
    assert np.array_equal(u8(packed), cases[2][3][0])


def test_static_scale_and_golden_vectors(device, golden):
    """The reference's own outputs (CPU ATen semantics = true division)."""
    for case in ("a", "b", "c", "d", "e"):
        xb = golden[f"{case}_x"]
        xd = torch.from_numpy(xb.copy()).view(torch.bfloat16).to(device)
        out = torch.empty(xb.shape, device=device, dtype=torch.uint8)
        scale = run_scale(xd, 448.0, 0)
        assert np.float32(scale.item()) == golden[f"{case}_fp8T_scale"]
        K.fp8_quantize(xd, out, scale, N.SPEC_T)
        assert np.array_equal(u8(out), golden[f"{case}_fp8T_codes"])
        K.fp8_quantize(xd, out, scale, N.SPEC_C)
        assert np.array_equal(u8(out), golden[f"{case}_fp8C_dyn_codes"])
        K.fp8_quantize(xd, out, torch.tensor(0.0371, device=device), N.SPEC_C)
        assert np.array_equal(u8(out), golden[f"{case}_fp8C_static_codes"])
        rows, columns = xb.shape
        packed = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
        linear = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8)
        blocked = torch.zeros(blocked_scale_bytes(rows, columns), device=device, dtype=torch.uint8)
        g = run_scale(xd, 2688.0, N.CLAMP_TINY)
        assert np.float32(g.item()) == golden[f"{case}_nv4T_global"]
        K.nvfp4_quantize(xd, packed, linear, blocked, g, N.SPEC_T)
        assert np.array_equal(u8(packed), golden[f"{case}_nv4T_packed"])
        assert np.array_equal(u8(linear), golden[f"{case}_nv4T_scales"])
        assert np.array_equal(u8(blocked), golden[f"{case}_nv4T_blocked"])


def test_every_bf16_value(device):
    """All 65,536 bf16 bit patterns (finite ones) through both encoders."""
    codes = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = np.isfinite(O.bf16_to_f32(codes))
    xb = codes[finite][: (finite.sum() // 64) * 64].reshape(-1, 64)
    xd = torch.from_numpy(xb.copy()).view(torch.bfloat16).to(device)
    for scale_value in (np.float32(1.0), np.float32(0.0371), np.float32(3.0e36)):
        scale = torch.tensor(float(scale_value), device=device)
        out = torch.empty(xb.shape, device=device, dtype=torch.uint8)
        K.fp8_quantize(xd, out, scale, N.SPEC_C)
        assert np.array_equal(u8(out), O.fp8_quantize_C(xb, scale_value)[0])
        K.fp8_quantize(xd, out, scale, N.SPEC_T | N.DIVISOR_BF16)
        assert np.array_equal(u8(out), O.fp8_quantize_T(xb, scale_value, divisor_bf16=True)[0])
    rows, columns = xb.shape
    packed = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8)
    for g_value in (np.float32(1.0), np.float32(2.5e-3), np.float32(1e30)):
        g = torch.tensor(float(g_value), device=device)
        K.nvfp4_quantize(xd, packed, linear, None, g, N.SPEC_C)
        want = O.nvfp4_quantize_C(xb, g_value)
        assert np.array_equal(u8(linear), want[1]) and np.array_equal(u8(packed), want[0])


def test_ragged_counts_and_zero_tensor(device):
    for count in (1, 7, 8, 9, 15, 4097):
        x = make_input((1, count), count, outliers=False)
        xd = x.to(device).reshape(-1)
        out = torch.full((count + 8,), 0x55, device=device, dtype=torch.uint8)
        scale = run_scale(xd, 448.0, N.SCALAR_RCP)
        K.fp8_quantize(xd, out[:count], scale, N.SPEC_C)
        want, want_scale = O.fp8_quantize_C(bits(x))
        assert np.float32(scale.item()) == want_scale
        assert np.array_equal(u8(out[:count]), want.reshape(-1))
        assert (u8(out[count:]) == 0x55).all(), "wrote past the end"
    zeros = torch.zeros((4, 64), device=device, dtype=torch.bfloat16)
    assert run_scale(zeros, 448.0, N.SCALAR_RCP).item() == 1.0
    assert np.float32(run_scale(zeros, 2688.0, N.CLAMP_TINY).item()) == O.nvfp4_global_scale(np.zeros((4, 64), np.float32), "T", "div")
    packed = torch.empty((4, 32), device=device, dtype=torch.uint8)
    K.nvfp4_quantize(zeros, packed, None, None, run_scale(zeros, 2688.0, N.CLAMP_TINY), N.SPEC_T)
    assert (u8(packed) == 0x77).all()          # the torch route encodes an all-zero block as code 7
    K.nvfp4_quantize(zeros, packed, None, None, run_scale(zeros, 2688.0, N.SCALAR_RCP), N.SPEC_C)
    assert (u8(packed) == 0).all()


def test_torch_cuda_semantics_of_the_reference_expressions(device):
    """What the reference's torch-route expressions evaluate to on a CUDA device
    (fp8.py:66-73 and nvfp4.py:28-46 restated with torch ops), against the flags the registry route uses."""
    x = make_input((130, 256), 77, 30.0)
    xb, xd = bits(x), x.to(device)
    peak = xd.float().abs().amax()
    scale = torch.where(peak > 0, peak / 448.0, torch.ones_like(peak))
    codes = (xd / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    mine = run_scale(xd, 448.0, N.SCALAR_RCP)
    assert mine.item() == scale.item()
    out = torch.empty(x.shape, device=device, dtype=torch.uint8)
    K.fp8_quantize(xd, out, mine, N.SPEC_T | N.DIVISOR_BF16)
    assert np.array_equal(u8(out), u8(codes))
    tiny = torch.finfo(torch.float32).tiny
    values = xd.float()
    g = values.abs().amax().clamp_min(tiny) / (448.0 * 6.0)
    grid = values.reshape(130, 16, 16)
    block = (grid.abs().amax(dim=-1) / 6.0 / g).clamp(tiny, 448.0).to(torch.float8_e4m3fn)
    scaled = (grid / (g * block.float()).unsqueeze(-1)).clamp(-6.0, 6.0).reshape(130, 256)
    thresholds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=device)
    nibbles = torch.bucketize(scaled.abs(), thresholds).to(torch.uint8) | ((scaled < 0).to(torch.uint8) << 3)
    want = (nibbles[:, 0::2] | (nibbles[:, 1::2] << 4)).contiguous()
    mine_g = run_scale(xd, 2688.0, N.SCALAR_RCP | N.CLAMP_TINY)
    assert mine_g.item() == g.item()
    packed = torch.empty((130, 128), device=device, dtype=torch.uint8)
    linear = torch.empty((130, 16), device=device, dtype=torch.uint8)
    K.nvfp4_quantize(xd, packed, linear, None, mine_g, N.SPEC_T | N.SCALAR_RCP)
    assert np.array_equal(u8(linear), u8(block)) and np.array_equal(u8(packed), u8(want))


def test_large_tensor_properties(device):
    """Rollout-sized tensor (17,920 x 2048): sign symmetry and agreement with per-slab encoding."""
    x = torch.randn((17920, 2048), device=device).to(torch.bfloat16)
    scale = run_scale(x, 448.0, N.SCALAR_RCP)
    assert scale.item() == (x.float().abs().amax() * (1.0 / 448.0)).item() or scale.item() == (x.float().abs().amax() / 448.0).item()
    full = torch.empty(x.shape, device=device, dtype=torch.uint8)
    K.fp8_quantize(x, full, scale, N.SPEC_C)
    negated = torch.empty_like(full)
    K.fp8_quantize(-x, negated, scale, N.SPEC_C)
    assert torch.equal(full ^ 0x80, negated)
    slab = torch.empty((560, 2048), device=device, dtype=torch.uint8)
    K.fp8_quantize(x[1120:1680].contiguous(), slab, scale, N.SPEC_C)
    assert torch.equal(slab, full[1120:1680])
    want = O.fp8_quantize_C(bits(x[:64]), np.float32(scale.item()))[0]
    assert np.array_equal(u8(full[:64]), want)


def test_division_by_repeated_divisor_is_correctly_rounded(device):
    """The encoders divide by a per-tensor / per-block constant through a reciprocal + one residual step;
    the codes must equal those of a true fp32 division for every bf16 dividend and for ordinary,
    extreme and all-ones-significand divisors."""
    rng = np.random.default_rng(5)
    codes = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = np.isfinite(O.bf16_to_f32(codes))
    xb = codes[finite][: (finite.sum() // 64) * 64].reshape(-1, 64)
    xd = torch.from_numpy(xb.copy()).view(torch.bfloat16).to(device)
    mantissas = rng.integers(0, 1 << 23, size=160, dtype=np.uint32)
    exponents = rng.integers(100, 150, size=160, dtype=np.uint32)
    scales = ((exponents << 23) | mantissas).view(np.float32).tolist()
    scales += [np.uint32(0x3F7FFFFF).view(np.float32).item(), np.uint32(0x3EFFFFFF).view(np.float32).item(),   # all ones
               1e-30, 1e30, 3.0e-39, 1.0, 0.5, 3.0, 7.0 / 448.0, float(np.float32(1.0) / np.float32(3.0))]
    out = torch.empty(xb.shape, device=device, dtype=torch.uint8)
    for value in scales:
        scale_value = np.float32(value)
        K.fp8_quantize(xd, out, torch.tensor(float(scale_value), device=device), N.SPEC_C)
        want = O.fp8_quantize_C(xb, scale_value)[0]
        assert np.array_equal(u8(out), want), f"scale {float(scale_value)!r}"
    rows, columns = xb.shape
    packed = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
    linear = torch.empty((rows, columns // 16), device=device, dtype=torch.uint8)
    for value in scales[:24] + scales[-10:-5]:
        g_value = np.float32(value)
        K.nvfp4_quantize(xd, packed, linear, None, torch.tensor(float(g_value), device=device), N.SPEC_C)
        want = O.nvfp4_quantize_C(xb, g_value)
        assert np.array_equal(u8(linear), want[1]) and np.array_equal(u8(packed), want[0]), f"global {float(g_value)!r}"
