"""The fused residual + RMSNorm + encoder kernel against the CPU oracle (oracle/norm_oracle.py), through the
C ABI.  The kernel's own reciprocal-root factor is read back, required to lie within 2 units in the last
place of the exactly rounded value of the oracle's kernel-order mean, and every other output must then be
bit-exact given that factor."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from embodiinfer_b200 import _native as N
from embodiinfer_b200 import kernels as K
from oracle import norm_oracle as NO
from tests.util import bits, u8

pytestmark = pytest.mark.gpu


def blocked_bytes(rows, blocks):
    return -(-rows // 128) * 128 * (-(-blocks // 4) * 4)


def run_case(device, *, batch, tokens, columns, bits_, adaptive, with_update, with_gate, given_mean=False, seed=0, flags=0):
    generator = torch.Generator().manual_seed(seed + columns + tokens)
    rows = batch * tokens
    inputs = (torch.randn((rows, columns), generator=generator) * 3).to(torch.bfloat16)
    inputs[0, :16] = 0
    update = torch.randn((rows, columns), generator=generator).to(torch.bfloat16) if with_update else None
    gate = torch.randn((batch, columns), generator=generator).to(torch.bfloat16) if with_gate else None
    scale = None if adaptive else torch.randn((columns,), generator=generator) * 0.2
    modulation = torch.randn((batch, 3 * columns), generator=generator) * 0.3 if adaptive else None
    mean = inputs.float().square().mean(dim=-1).contiguous() if given_mean else None
    global_scale = torch.tensor({8: 0.011, 4: 0.0023, 16: 1.0}[bits_])
    to = lambda t: None if t is None else t.to(device)
    width = {16: 2 * columns, 8: columns, 4: columns // 2}[bits_]
    output = torch.zeros((rows, width), device=device, dtype=torch.uint8)
    residual = torch.zeros((rows, columns), device=device, dtype=torch.bfloat16)
    scales = torch.zeros((rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
    next_gate = torch.zeros((batch, columns), device=device, dtype=torch.bfloat16) if adaptive else None
    inverse = torch.zeros(rows, device=device)
    K.norm_quant(to(inputs), output, bits=bits_, tokens=tokens, scale=to(scale), modulation=to(modulation), update=to(update),
                 update_gate=to(gate), mean=to(mean), global_scale=None if bits_ == 16 else to(global_scale),
                 residual=residual, scales=scales, blocked=blocked, gate=next_gate, inverse=inverse, flags=flags)
    torch.cuda.synchronize()
    np_or_none = lambda t: None if t is None else t.numpy()
    expected = NO.norm_quant(bits(inputs), bits=bits_, tokens=tokens, scale=np_or_none(scale), modulation=np_or_none(modulation),
                             update=None if update is None else bits(update), update_gate=None if gate is None else bits(gate),
                             mean=np_or_none(mean), global_scale=np.float32(global_scale.item()), inverse=inverse.cpu().numpy())
    assert np.all(NO.ulp_distance(inverse.cpu().numpy(), NO.inverse_exact(expected["term"])) <= 2)
    assert np.array_equal(bits(residual), expected["residual"])
    got = u8(output)
    want = expected["output"].view(np.uint8).reshape(rows, -1)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} output bytes differ"
    if bits_ == 4:
        assert np.array_equal(u8(scales), expected["scales"])
        assert np.array_equal(u8(blocked), expected["blocked"].reshape(-1))
    if adaptive:
        assert np.array_equal(bits(next_gate), expected["gate"])


@pytest.mark.parametrize("bits_", [8, 4, 16])
@pytest.mark.parametrize("columns", [2048, 1024])
def test_rms_norm_encode_lane_order(device, bits_, columns):
    run_case(device, batch=2, tokens=35, columns=columns, bits_=bits_, adaptive=False, with_update=False, with_gate=False)
    run_case(device, batch=2, tokens=35, columns=columns, bits_=bits_, adaptive=False, with_update=True, with_gate=False, seed=1)


@pytest.mark.parametrize("bits_", [8, 4, 16])
def test_adaptive_modulation_and_gated_update(device, bits_):
    run_case(device, batch=3, tokens=10, columns=1024, bits_=bits_, adaptive=True, with_update=True, with_gate=True, seed=2)
    run_case(device, batch=3, tokens=10, columns=1024, bits_=bits_, adaptive=True, with_update=False, with_gate=False, seed=3)


@pytest.mark.parametrize("bits_", [8, 4, 16])
@pytest.mark.parametrize("columns", [64, 1152, 4096, 8192])
def test_strided_order_widths(device, bits_, columns):
    run_case(device, batch=2, tokens=9, columns=columns, bits_=bits_, adaptive=False, with_update=True, with_gate=False, seed=4)
    run_case(device, batch=2, tokens=3, columns=columns, bits_=bits_, adaptive=True, with_update=True, with_gate=True, seed=5)


@pytest.mark.parametrize("bits_", [8, 4])
def test_given_mean_divides_by_the_scale(device, bits_):
    run_case(device, batch=2, tokens=17, columns=2048, bits_=bits_, adaptive=False, with_update=False, with_gate=False,
             given_mean=True, seed=6)
    run_case(device, batch=2, tokens=5, columns=320, bits_=bits_, adaptive=True, with_update=False, with_gate=False,
             given_mean=True, seed=7)


def test_full_prefix_micro_batch_and_evict_last(device):
    """The rollout's shape (32 observations x 560 tokens x 2048), with the residual stored evict-last."""
    run_case(device, batch=32, tokens=560, columns=2048, bits_=8, adaptive=False, with_update=True, with_gate=False, seed=8,
             flags=N.NORM_RESIDUAL_EVICT_LAST)


@pytest.mark.parametrize("bits_", [8, 4, 16])
def test_row_per_warp_variants(device, bits_):
    """4096 rows and more run one warp per row; same results as the oracle in every mode."""
    run_case(device, batch=5, tokens=840, columns=1024, bits_=bits_, adaptive=True, with_update=True, with_gate=True, seed=9)
    run_case(device, batch=2, tokens=2100, columns=2048, bits_=bits_, adaptive=False, with_update=False, with_gate=False, seed=10)
    if bits_ != 16:
        run_case(device, batch=1, tokens=4099, columns=1024, bits_=bits_, adaptive=False, with_update=False, with_gate=False,
                 given_mean=True, seed=11)


def test_rejects_bad_arguments(device):
    x = torch.zeros((4, 64), device=device, dtype=torch.bfloat16)
    out = torch.zeros((4, 64), device=device, dtype=torch.uint8)
    scale = torch.zeros(64, device=device)
    g = torch.ones((), device=device)
    with pytest.raises(RuntimeError):      # neither scale nor modulation
        K.norm_quant(x, out, bits=8, tokens=4, global_scale=g)
    with pytest.raises(RuntimeError):      # rows not a multiple of tokens
        K.norm_quant(x, out, bits=8, tokens=3, scale=scale, global_scale=g)
    with pytest.raises(RuntimeError):      # unsupported bit width
        K.norm_quant(x, out, bits=6, tokens=4, scale=scale, global_scale=g)
    with pytest.raises(RuntimeError):      # NVFP4 needs the tiled scale buffer
        K.norm_quant(x, out, bits=4, tokens=4, scale=scale, global_scale=g)
    narrow = torch.zeros((4, 48), device=device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):      # width must be a multiple of 64
        K.norm_quant(narrow, out, bits=8, tokens=4, scale=scale, global_scale=g)


def run_layer_norm(device, *, rows, columns, bits_, with_update, seed):
    generator = torch.Generator().manual_seed(seed + columns)
    inputs = (torch.randn((rows, columns), generator=generator) * 2 + 0.3).to(torch.bfloat16)
    inputs[0, :16] = 0
    update = torch.randn((rows, columns), generator=generator).to(torch.bfloat16) if with_update else None
    weight = torch.randn((columns,), generator=generator).to(torch.bfloat16)
    bias = torch.randn((columns,), generator=generator).to(torch.bfloat16)
    scale_value = {8: 448.0 / 11.0, 4: 11.0 / 2688.0, 16: 1.0}[bits_]
    width = {16: 2 * columns, 8: columns, 4: columns // 2}[bits_]
    output = torch.zeros((rows, width), device=device, dtype=torch.uint8)
    residual = torch.zeros((rows, columns), device=device, dtype=torch.bfloat16)
    scales = torch.zeros((rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
    blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
    statistics = torch.zeros((rows, 2), device=device)
    K.layer_norm_quant(inputs.to(device), weight.to(device), bias.to(device), output, bits=bits_, scale_value=scale_value,
                       update=None if update is None else update.to(device), residual=residual, scales=scales, blocked=blocked,
                       statistics=statistics)
    torch.cuda.synchronize()
    measured = statistics.cpu().numpy()
    expected = NO.layer_norm_quant(bits(inputs), bits(weight), bits(bias), bits=bits_, scale_value=np.float32(scale_value),
                                   update=None if update is None else bits(update), deviation=measured[:, 1])
    assert np.array_equal(measured[:, 0], expected["mean"])
    assert np.all(NO.ulp_distance(measured[:, 1], NO.inverse_exact(expected["term"])) <= 2)
    assert np.array_equal(bits(residual), expected["residual"])
    got, want = u8(output), expected["output"].view(np.uint8).reshape(rows, -1)
    assert np.array_equal(got, want), f"{(got != want).sum()} of {got.size} output bytes differ"
    if bits_ == 4:
        assert np.array_equal(u8(scales), expected["scales"])
        assert np.array_equal(u8(blocked), expected["blocked"].reshape(-1))


@pytest.mark.parametrize("bits_", [8, 4, 16])
@pytest.mark.parametrize("columns", [1152, 2048, 64, 1024, 1168])
def test_layer_norm_encode(device, bits_, columns):
    run_layer_norm(device, rows=37, columns=columns, bits_=bits_, with_update=True, seed=20)
    run_layer_norm(device, rows=130, columns=columns, bits_=bits_, with_update=False, seed=21)


@pytest.mark.parametrize("bits_", [8, 4, 16])
def test_layer_norm_row_per_warp(device, bits_):
    run_layer_norm(device, rows=4100, columns=1152, bits_=bits_, with_update=True, seed=22)
    run_layer_norm(device, rows=4096, columns=2048, bits_=bits_, with_update=False, seed=23)


def test_layer_norm_rejects_bad_arguments(device):
    x = torch.zeros((4, 64), device=device, dtype=torch.bfloat16)
    w = torch.zeros(64, device=device, dtype=torch.bfloat16)
    out = torch.zeros((4, 64), device=device, dtype=torch.uint8)
    with pytest.raises(RuntimeError):      # NVFP4 needs the tiled scale buffer
        K.layer_norm_quant(x, w, w, out, bits=4, scale_value=0.01)
    with pytest.raises(RuntimeError):      # the e4m3 multiplier must be positive
        K.layer_norm_quant(x, w, w, out, bits=8, scale_value=0.0)
    wide = torch.zeros((2, 4096), device=device, dtype=torch.bfloat16)
    wide_w = torch.zeros(4096, device=device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):      # beyond the 256-thread block of the reference
        K.layer_norm_quant(wide, wide_w, wide_w, torch.zeros((2, 4096), device=device, dtype=torch.uint8), bits=8, scale_value=1.0)


@pytest.mark.parametrize("bits_", [8, 4, 16])
@pytest.mark.parametrize("batch,heads,tokens,head_dim", [(1, 8, 560, 256), (3, 8, 10, 256), (2, 16, 256, 72), (2, 3, 5, 16)])
def test_attention_output_transposing_encoder(device, bits_, batch, heads, tokens, head_dim):
    if bits_ == 4 and head_dim % 16:
        pytest.skip("NVFP4 blocks need head_dim % 16 == 0")
    generator = torch.Generator().manual_seed(head_dim + tokens)
    attended = (torch.randn((batch, heads, tokens, head_dim), generator=generator) * 2).to(torch.bfloat16)
    attended[0, 0, 0, :16] = 0
    rows, columns = batch * tokens, heads * head_dim
    scale_value = {8: 448.0 / 9.0, 4: 9.0 / 2688.0, 16: 1.0}[bits_]
    width = {16: 2 * columns, 8: columns, 4: columns // 2}[bits_]
    expected = NO.bhsd_quant(bits(attended), bits_, np.float32(scale_value))
    # contiguous [B, H, S, D], and the same values held as a transposed view of [B, S, H, D]
    for source in (attended.to(device), attended.to(device).transpose(1, 2).contiguous().transpose(1, 2)):
        output = torch.zeros((rows, width), device=device, dtype=torch.uint8)
        scales = torch.zeros((rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
        blocked = torch.zeros(blocked_bytes(rows, columns // 16), device=device, dtype=torch.uint8) if bits_ == 4 else None
        K.bhsd_quant(source, output, bits=bits_, scale_value=scale_value, scales=scales, blocked=blocked)
        torch.cuda.synchronize()
        assert np.array_equal(u8(output), expected["output"].view(np.uint8).reshape(rows, -1))
        if bits_ == 4:
            assert np.array_equal(u8(scales), expected["scales"])
            assert np.array_equal(u8(blocked), expected["blocked"].reshape(-1))
