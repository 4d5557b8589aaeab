"""Weight bundles: buffer names / dtypes / shapes of the reference, values against the oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from torch import nn

from embodiinfer_b200 import weights as W
from embodiinfer_b200.bundles import FP8Linear, NVFP4Linear, pack_quantized_linears, quantize_linear
from embodiinfer_b200.layers import FP8Config, NVFP4Config
from oracle import quant_oracle as O
from tests.util import make_weight, u8


def linear(n, k, seed, bias=False):
    module = nn.Linear(k, n, bias=bias)
    module.weight.data = make_weight((n, k), seed)
    return module


def test_fp8_bundle_layout_and_values(golden):
    module = quantize_linear(linear(48, 64, 1), FP8Config(scaling_scheme="tensorwise"))
    state = module.state_dict()
    assert sorted(state) == ["weight", "weight_scale"]
    assert state["weight"].dtype == torch.uint8 and state["weight"].shape == (48, 64)
    assert state["weight_scale"].dtype == torch.float32 and state["weight_scale"].shape == ()
    assert module.quantized_weight.dtype == torch.float8_e4m3fn
    codes, scale = O.fp8_quantize_weight_tensorwise(make_weight((48, 64), 1).numpy(), "div")
    assert np.array_equal(u8(state["weight"]), codes) and float(state["weight_scale"]) == float(scale)
    channel = quantize_linear(linear(48, 64, 1), FP8Config(scaling_scheme="channelwise"))
    assert channel.weight_scale.shape == (48,)
    # golden weights produced by the reference itself
    w = torch.from_numpy(golden["a_w"])
    codes, scale = W.fp8_quantize_tensorwise(w)
    assert np.array_equal(u8(codes), golden["a_wfp8_codes"]) and float(scale) == float(golden["a_wfp8_scale"])


def test_nvfp4_bundle_layout_and_values(golden):
    module = quantize_linear(linear(130, 64, 2, bias=True), NVFP4Config())
    state = module.state_dict()
    assert sorted(state) == ["bias", "quantization_thresholds", "weight", "weight_global_scale", "weight_scale", "weight_scale_blocked"]
    assert state["weight"].shape == (130, 32) and state["weight"].dtype == torch.uint8
    assert state["weight_scale"].shape == (130, 4) and state["weight_scale"].dtype == torch.uint8
    assert state["weight_scale_blocked"].shape == (2 * 512,) and state["weight_scale_blocked"].dtype == torch.uint8
    assert state["weight_global_scale"].shape == () and state["weight_global_scale"].dtype == torch.float32
    assert state["quantization_thresholds"].tolist() == [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    packed, scales, g = O.nvfp4_quantize_T(make_weight((130, 64), 2).numpy(), "div", is_bf16=False)
    assert np.array_equal(u8(state["weight"]), packed) and np.array_equal(u8(state["weight_scale"]), scales)
    assert float(state["weight_global_scale"]) == float(g)
    assert np.array_equal(u8(state["weight_scale_blocked"]), O.swizzle_scales(scales))
    for case in ("a", "b", "e"):
        w = torch.from_numpy(golden[f"{case}_w"])
        packed, scales, g = W.nvfp4_quantize_weight(w)
        assert np.array_equal(u8(packed), golden[f"{case}_wnv4_packed"])
        assert np.array_equal(u8(scales), golden[f"{case}_wnv4_scales"])
        assert float(g) == float(golden[f"{case}_wnv4_global"])


@pytest.mark.parametrize("config", (FP8Config(scaling_scheme="tensorwise"), NVFP4Config()))
def test_pack_shares_storage_and_one_scale(config):
    members = tuple(quantize_linear(linear(n, 64, 10 + n), config) for n in (32, 16, 16))
    packed = pack_quantized_linears(members)
    assert packed.out_features == 64 and packed.split_sizes == (32, 16, 16)
    begin = 0
    for member in members:
        assert member.weight.data_ptr() == packed.weight[begin:].data_ptr()
        begin += member.out_features
    if isinstance(config, FP8Config):
        assert all(m.weight_scale is packed.weight_scale for m in members)
    else:
        assert all(m.weight_global_scale is packed.weight_global_scale for m in members)
        assert members[1].weight_scale_blocked.numel() == 512
    with pytest.raises(ValueError, match="empty"):
        pack_quantized_linears(())
    with pytest.raises(ValueError, match="same quantization method"):
        pack_quantized_linears((members[0], quantize_linear(linear(8, 64, 3), FP8Config() if isinstance(config, NVFP4Config) else NVFP4Config())))
    with pytest.raises(ValueError):
        type(packed).pack((members[0], quantize_linear(linear(8, 64, 3, bias=True), config)))


def test_cast_keeps_fp32_metadata():
    module = quantize_linear(linear(16, 64, 5).to(torch.bfloat16), NVFP4Config())
    before = module.weight_global_scale.clone()
    module = module.to(torch.float16)
    assert module.weight_global_scale.dtype == torch.float32 and torch.equal(module.weight_global_scale, before)
    assert module.quantization_thresholds.dtype == torch.float32 and module.compute_dtype == torch.float16
    fp8 = quantize_linear(linear(16, 64, 5).to(torch.bfloat16), FP8Config(scaling_scheme="tensorwise")).to(torch.bfloat16)
    assert fp8.weight_scale.dtype == torch.float32


def test_forward_rejects_wrong_width_and_cpu_has_no_fallback():
    module = quantize_linear(linear(16, 64, 6), FP8Config(scaling_scheme="tensorwise"))
    with pytest.raises(ValueError, match="expected K=64"):
        module(torch.zeros(2, 32))
    with pytest.raises(RuntimeError, match="no CPU or weight-only fallback"):
        module(torch.zeros(2, 64, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="cannot FP8-quantize"):
        FP8Linear.from_linear(nn.ReLU(), FP8Config())
    with pytest.raises(ValueError, match="scalar or per-channel"):
        FP8Linear(torch.zeros(4, 16, dtype=torch.uint8), torch.ones(3), None, compute_dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="one weight scale per 16"):
        NVFP4Linear(torch.zeros(4, 16, dtype=torch.uint8), torch.zeros(4, 3, dtype=torch.uint8), torch.ones(()), None, compute_dtype=torch.bfloat16)


def test_dequantise_round_trip(golden):
    w = torch.from_numpy(golden["a_w"])
    packed, scales, g = W.nvfp4_quantize_weight(w)
    dense = W.nvfp4_dequantize_weight(packed, scales, g, torch.float32).numpy()
    assert np.array_equal(dense, O.nvfp4_dequantize(u8(packed), u8(scales), np.float32(g.item())))
    # requantising an NVFP4-representable matrix reproduces its values (the sign of a zero code may differ)
    again = W.nvfp4_quantize_weight(torch.from_numpy(dense))
    assert np.array_equal(W.nvfp4_dequantize_weight(*again, torch.float32).numpy(), dense)
