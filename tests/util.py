"""Helpers shared by the tests: seeded inputs (the same recipe as tests/golden/make_golden.py),
bit views, and the parity tolerances."""

from __future__ import annotations

import numpy as np
import torch

from oracle import quant_oracle as O

# Tolerances for GEMM / layer outputs in bf16 against the reference's result on identical
# quantised operands.
REL_FROBENIUS = 1e-3
MAX_ABS = 2e-2


def make_input(shape, seed, multiplier=1.0, outliers=True):
    """bf16 activations ~N(0,1)*multiplier with 1% outliers x20, a zero block and a signed-zero block."""
    generator = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=generator) * multiplier
    if outliers:
        x = torch.where(torch.rand(shape, generator=generator) < 0.01, x * 20, x)
    else:
        torch.rand(shape, generator=generator)
    x = x.to(torch.bfloat16)
    if len(shape) == 2 and shape[0] > 1 and shape[1] >= 32:
        x[0, :16] = 0
        x[1, 16:32] = torch.tensor([0.0, -0.0] * 8).to(torch.bfloat16)
    return x


def make_weight(shape, seed, std=0.02):
    generator = torch.Generator().manual_seed(seed + 5000)
    return torch.randn(shape, generator=generator) * std


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().cpu().contiguous().view(torch.uint16).numpy()


def u8(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().cpu().contiguous().view(torch.uint8).numpy()


def assert_gemm_close(got_bf16: np.ndarray, want_bf16: np.ndarray) -> None:
    """rel-Frobenius <= 1e-3 and max-abs <= 2e-2 in bf16.

    One bf16 unit in the last place is 2^-8 relative, i.e. already 3.1e-2 for a value in [4, 8):
    two correct fp32 accumulations in different orders can land on adjacent bf16 values.  Where the
    expected magnitude makes one ulp exceed 2e-2 the per-element bound is therefore one ulp of the
    expected value; below that it is the absolute 2e-2.
    """
    assert got_bf16.shape == want_bf16.shape
    got = O.bf16_to_f32(got_bf16).astype(np.float64)
    want = O.bf16_to_f32(want_bf16).astype(np.float64)
    assert np.isfinite(got).all()
    assert O.rel_frobenius(got_bf16, want_bf16) <= REL_FROBENIUS
    ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(want), 1e-30))) - 7)
    bound = np.maximum(MAX_ABS, ulp)
    worst = np.abs(got - want) - bound
    assert worst.max() <= 0, f"max-abs violation {np.abs(got - want).max()}"


def _bf16_neighbours(bits16: np.ndarray) -> list[np.ndarray]:
    """The bf16 value itself and the two adjacent bf16 values (one unit in the last place either way)."""
    b = bits16.astype(np.int32)
    magnitude = b & 0x7FFF
    up = np.where(magnitude < 0x7F7F, b + 1, b)
    down = np.where(magnitude > 0, b - 1, (b ^ 0x8000) | 1)       # below +-0 lies the smallest value of the other sign
    return [bits16, up.astype(np.uint16), down.astype(np.uint16)]


def assert_gated_close(got_bf16: np.ndarray, gate_bf16: np.ndarray, up_bf16: np.ndarray, table_u16: np.ndarray) -> None:
    """The fused gated epilogue against the oracle's gate and up projections.

    h = bf16(bf16(gelu(gate)) * up) amplifies a one-ulp difference of gate or up (two correct fp32 accumulation orders
    can round to adjacent bf16 values) by the other factor, so a bound on |h - h_oracle| alone says little.  Instead
    every element must EQUAL the oracle's h for some gate and some up each within one bf16 ulp of the oracle's, at
    least 99 % must be the oracle's own h, and the whole tensor must stay within the relative Frobenius bound."""
    assert got_bf16.shape == gate_bf16.shape == up_bf16.shape
    assert O.rel_frobenius(got_bf16, O.gelu_mul(gate_bf16, up_bf16, table_u16)) <= REL_FROBENIUS
    central = got_bf16 == O.gelu_mul(gate_bf16, up_bf16, table_u16)
    matched = central.copy()
    for gate in _bf16_neighbours(gate_bf16):
        for up in _bf16_neighbours(up_bf16):
            matched |= got_bf16 == O.gelu_mul(gate, up, table_u16)
    assert matched.all(), f"{(~matched).sum()} of {matched.size} elements are no neighbour's result"
    assert central.mean() >= 0.99, f"only {central.mean():.4f} of the elements are the oracle's own result"


def gelu_table_cpu(approximate="tanh") -> np.ndarray:
    codes = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16)
    return torch.nn.functional.gelu(codes, approximate=approximate).view(torch.uint16).numpy()
