"""The reference-facing API on the GPU: registry Linear (bundles), plan registries, fused MLP.
Mirrors the reference's own GPU tests for this path (tests/test_fused_operators.py:125-298,
tests/pi05/test_graphs.py:238-313): fused == separate bit for bit, graph replay == eager."""

from __future__ import annotations

import numpy as np
import pytest
import torch
from torch import nn

from embodiinfer_b200 import layers as L
from embodiinfer_b200.backend.mlp import FusedMlpPlan
from embodiinfer_b200.bundles import pack_quantized_linears, quantize_linear
from embodiinfer_b200.layers.registry import OperatorRequest
from oracle import quant_oracle as O
from tests.util import assert_gemm_close, bits, gelu_table_cpu, make_input, make_weight, u8

pytestmark = pytest.mark.gpu


def request(device, shape=None, bits_=None):
    return OperatorRequest(device, torch.bfloat16, shape=shape, bits=bits_, cuda_graph=True)


def module(n, k, seed, device, bias=False):
    layer = nn.Linear(k, n, bias=bias)
    layer.weight.data = make_weight((n, k), seed)
    if bias:
        layer.bias.data = make_weight((1, n), seed + 1, std=0.1).reshape(-1)
    return layer.to(device=device, dtype=torch.bfloat16)


def test_fp8_registry_linear_matches_reference_route(device):
    """FP8Linear.forward -> fp8_native: oracle spec T with CUDA ATen semantics + W8A8 GEMM + bias."""
    layer = module(1024, 2048, 3, device, bias=True)
    bundle = quantize_linear(layer, L.FP8Config(backend="native"))
    assert bundle.weight_scale.ndim == 0          # tensorwise on Blackwell (fp8.py:80-85)
    x = make_input((2, 40, 2048), 5).to(device)
    y = bundle(x)
    assert y.shape == (2, 40, 1024) and y.dtype == torch.bfloat16
    xb = bits(x).reshape(80, 2048)
    aq, a_s = O.fp8_quantize_T(xb, scalar_div="rcp", divisor_bf16=True)
    want = O.fp8_linear(aq, a_s, u8(bundle.weight), np.float32(bundle.weight_scale.item()), bits(layer.bias))
    assert_gemm_close(bits(y).reshape(80, 1024), want)
    # weight codes equal the oracle's weight quantiser under CUDA ATen semantics
    codes, scale = O.fp8_quantize_weight_tensorwise(O.bf16_to_f32(bits(layer.weight)), "rcp")
    assert np.array_equal(u8(bundle.weight), codes) and np.float32(bundle.weight_scale.item()) == scale


def test_nvfp4_registry_linear_and_pack(device):
    q, k, v = (module(n, 2048, 10 + i, device) for i, n in enumerate((2048, 256, 256)))
    members = tuple(quantize_linear(layer, L.NVFP4Config(backend="auto")) for layer in (q, k, v))
    packed = pack_quantized_linears(members)
    x = make_input((560, 2048), 6).to(device)
    y = packed(x)
    assert y.shape == (560, 2560)
    ap, asl, a_g = O.nvfp4_quantize_T(bits(x), "rcp")
    want = O.nvfp4_linear_registry(ap, asl, a_g, u8(packed.weight), u8(packed.weight_scale),
                                   np.float32(packed.weight_global_scale.item()))
    assert_gemm_close(bits(y), want)
    # a member views the packed storage, so it gives the matching slice
    assert torch.equal(members[1](x), y[:, 2048:2304])


def test_explicit_backend_errors(device):
    layer = module(64, 72, 1, device)       # K = 72 is not a multiple of 16
    with pytest.raises(RuntimeError, match="K divisible by 16"):
        quantize_linear(layer, L.FP8Config(backend="native", scaling_scheme="tensorwise"))(torch.zeros((4, 72), device=device, dtype=torch.bfloat16))
    channel = quantize_linear(module(64, 64, 1, device), L.FP8Config(backend="native", scaling_scheme="channelwise"))
    with pytest.raises(RuntimeError, match="requires tensorwise weights"):
        channel(torch.zeros((4, 64), device=device, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU or weight-only fallback"):
        quantize_linear(module(64, 64, 1, device), L.FP8Config(backend="torch"))(torch.zeros((4, 64), device=device, dtype=torch.bfloat16))


def test_quantizer_plans(device):
    quantizer = L.quantization_backends.get("cuda", request(device, (560, 2048), 8))
    x = make_input((560, 2048), 8).to(device)
    plan = quantizer.plan(x, 8)
    assert plan.dynamic and plan.quantize(x) is plan
    codes, scale = O.fp8_quantize_C(bits(x))
    assert np.float32(plan.scale.item()) == scale and np.array_equal(u8(plan.output), codes)
    static = quantizer.plan(x, 4, 0.0123).quantize(x)
    want = O.nvfp4_quantize_C(bits(x), np.float32(0.0123))
    assert np.array_equal(u8(static.output), want[0]) and np.array_equal(u8(static.scales), want[1])
    assert np.array_equal(u8(static.blocked), want[2]) and static.output.shape == (560, 1024)
    with pytest.raises(ValueError, match="K divisible by 64"):
        quantizer.plan(torch.zeros((4, 48), device=device, dtype=torch.bfloat16), 8)
    with pytest.raises(ValueError, match="finite and positive"):
        quantizer.plan(x, 8, float("nan"))
    with pytest.raises(ValueError, match="contiguous CUDA BF16"):
        quantizer.plan(x.float(), 8)
    with pytest.raises(ValueError, match="shape or layout changed"):
        plan.quantize(x[:100])
    with pytest.raises(ValueError, match="3-bit"):
        L.quantization_backends.get("cuda", request(device, (8, 64), 3))


@pytest.mark.parametrize("bits_", (16, 8, 4))
def test_standalone_gelu_mul_equals_separate_steps(device, bits_):
    quantizer = L.quantization_backends.get("cuda", request(device))
    fusion = L.gelu_mul_backends.get("cuda", request(device), backend=quantizer, approximate="tanh")
    gate, up = make_input((130, 256), 1).to(device), make_input((130, 256), 2, outliers=False).to(device)
    # The table is the framework's GELU evaluated on the device (activation.py:34-37); NaN inputs aside
    # it must agree with the CPU evaluation that the golden vectors were made with.
    table = u8(fusion.table).view(np.uint16)
    finite = np.isfinite(O.bf16_to_f32(np.arange(65536, dtype=np.uint32).astype(np.uint16)))
    cpu_table = gelu_table_cpu("tanh")
    differing = np.nonzero(finite & (table != cpu_table))[0]
    # The device's tanh and the host's differ for a handful of inputs (on a B200 with torch 2.11: the four
    # codes 0xc0a2..0xc0a5, x ~ -5.1, where the host saturates tanh to -1 and returns -0.0 while the device
    # returns -1.5e-7); the kernels take the table as an operand, so either one is reproduced exactly.
    assert len(differing) <= 16
    on_device, on_host = O.bf16_to_f32(table[differing]), O.bf16_to_f32(cpu_table[differing])
    close = np.abs(on_device - on_host) <= 1e-6 + 2.0**-7 * np.maximum(np.abs(on_device), np.abs(on_host))
    assert close.all(), [(hex(int(c)), float(a), float(b)) for c, a, b in zip(differing, on_device, on_host)]
    hidden = O.gelu_mul(bits(gate), bits(up), table)
    scale = None if bits_ == 16 else 0.05
    plan = fusion.plan(gate, bits_, scale).encode(gate, up)
    if bits_ == 16:
        assert np.array_equal(bits(plan.output), hidden)
        packed = fusion.plan(gate, 16).encode_packed(torch.cat((gate, up), dim=1).contiguous())
        assert np.array_equal(bits(packed.output), hidden)
    elif bits_ == 8:
        want = O.e4m3_encode_satfinite((O.bf16_to_f32(hidden) * (np.float32(1.0) / np.float32(0.05))).astype(np.float32))
        assert np.array_equal(u8(plan.output), want)
    else:
        want = O.nvfp4_quantize_C(hidden, np.float32(0.05))
        assert np.array_equal(u8(plan.output), want[0]) and np.array_equal(u8(plan.scales), want[1])
        assert np.array_equal(u8(plan.blocked), want[2])


@pytest.mark.parametrize("precision", ("fp8", "nvfp4"))
def test_projection_plan_and_fused_mlp(device, precision):
    """Fused MLP (3 launches) == encode, gate GEMM, up GEMM, stand-alone GELU*up encode, down GEMM."""
    hidden_size, inter = 1024, 4096
    quantizer = L.quantization_backends.get("cuda", request(device))
    projections = L.projection_backends.get("cuda", request(device))
    fusion = L.gelu_mul_backends.get("cuda", request(device), backend=quantizer, approximate="tanh")
    gate_w, up_w = (make_weight((inter, hidden_size), s).to(device, torch.bfloat16) for s in (1, 2))
    down_w = make_weight((hidden_size, inter), 3).to(device, torch.bfloat16)
    x = make_input((1, 560, hidden_size), 4).to(device)
    key = lambda dev: ("stream", torch.cuda.current_stream(dev).cuda_stream)
    gate = projections.plan(gate_w, 40.0, precision, quantizer, key)
    up = projections.plan(up_w, 40.0, precision, quantizer, key)
    down = projections.plan(down_w, 8.0, precision, quantizer, key)
    encoded = gate.encode(x)
    g, u = gate.apply(x, encoded), up.apply(x, encoded)
    assert g.shape == (1, 560, inter)
    # oracle check of one projection
    xb = bits(x).reshape(560, hidden_size)
    if precision == "fp8":
        aq, a_s = O.fp8_quantize_C(xb, np.float32(40.0 / 448))
        want = O.fp8_linear(aq, a_s, u8(gate.weight), np.float32(gate.weight_scale.item()))
    else:
        ap, asl, _, a_s = O.nvfp4_quantize_C(xb, np.float32(40.0 / 2688))
        wp, wsl, _, w_s = O.nvfp4_quantize_C(bits(gate_w))
        assert np.array_equal(u8(gate.weight), wp) and np.float32(gate.weight_scale.item()) == w_s
        want = O.nvfp4_linear_plan(ap, asl, a_s, wp, wsl, w_s)
    assert_gemm_close(bits(g).reshape(560, inter), want)
    bits_ = 8 if precision == "fp8" else 4
    separate = fusion.plan(g.reshape(560, inter), bits_, 8.0 / (448 * (6 if bits_ == 4 else 1)))
    separate.encode(g.reshape(560, inter), u.reshape(560, inter).contiguous())
    y_separate = down.apply(g, separate).clone()
    mlp = FusedMlpPlan(gate_w, up_w, down_w, gate_up_max=40.0, down_max=8.0, gate_up=precision, down=precision,
                       quantizer=quantizer, approximate="tanh", workspace_key=key)
    y_fused = mlp(x)
    assert torch.equal(y_fused, y_separate), "fused MLP differs from the separate steps"
    residual = make_input((1, 560, hidden_size), 9, outliers=False).to(device)
    assert torch.equal(mlp(x, residual=residual), y_separate + residual)
    # graph replay == eager (after the warm-up above)
    static_x = x.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        mlp(static_x)                              # warm this stream's workspaces
        with torch.cuda.graph(graph, stream=side):
            y_graph = mlp(static_x)
    static_x.copy_(make_input((1, 560, hidden_size), 44).to(device))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_graph, mlp(static_x))
    scope = key(device)
    mlp.release_scope(scope)
    assert all(k[-1] != scope for k in (*mlp.gate_up.plans, *mlp.gate_up.outputs, *mlp.down.outputs))


def test_backend_construction_refused_during_capture(device):
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with pytest.raises(RuntimeError, match="before CUDA Graph capture"):
            with torch.cuda.graph(graph, stream=side):
                L.quantization_backends.get("cuda", request(device))


@pytest.mark.parametrize("precision", ["fp8", "nvfp4"])
def test_calibrated_layer_record_with_smoothquant_scales(device, precision):
    """A layer record with SmoothQuant scales: gate/up are packed as W*s and the caller feeds x/s (the folded norm),
    so the fused MLP's result stays that of the unsmoothed plan up to quantisation noise; the fused norm + encoder
    launch with the folded norm scale produces the x/s encoding directly."""
    from embodiinfer_b200 import calibration as C
    from embodiinfer_b200.backend.norm_quant import B200NormQuant
    from embodiinfer_b200.backend.quantization import B200Quantizer
    hidden_size, inter = 256, 512
    quantizer = B200Quantizer()
    gate_w, up_w = make_weight((inter, hidden_size), 61).bfloat16().to(device), make_weight((inter, hidden_size), 62).bfloat16().to(device)
    down_w = make_weight((hidden_size, inter), 63).bfloat16().to(device)
    generator = torch.Generator().manual_seed(64)
    smooth = (torch.rand(hidden_size, generator=generator) * 1.5 + 0.5)
    residual = make_input((1, 70, hidden_size), 65, outliers=False).to(device)
    norm_weight = (torch.randn(hidden_size, generator=generator) * 0.1).to(device)
    inverse = torch.rsqrt(residual.float().square().mean(-1, keepdim=True) + 1e-6)
    normed = (residual.float() * inverse * (1 + norm_weight)).to(torch.bfloat16)
    plain = C.fused_mlp_from_layer(gate_w, up_w, down_w, C.MlpLayerPrecision(precision, precision, 8.0, 2.0), quantizer)
    expected = plain(normed.reshape(70, hidden_size))
    layer = C.MlpLayerPrecision(precision, precision, 16.0, 2.0, smooth=[float(v) for v in smooth])
    smoothed = C.fused_mlp_from_layer(gate_w, up_w, down_w, layer, quantizer)
    folded_scale = C.smoothed_norm_scale(norm_weight, smooth.to(device))
    bits_ = 8 if precision == "fp8" else 4
    plan = B200NormQuant(quantizer).plan(residual, bits=bits_, calibrated_scale=16.0 / (448 * (6 if bits_ == 4 else 1)), adaptive=False)
    encoded = plan.normalize(residual, scale=folded_scale)
    got = smoothed.project(residual.reshape(70, hidden_size), encoded)
    # both plans carry their own quantisation noise: measure each against the unquantised MLP on the same input
    n = normed.reshape(70, hidden_size).float()
    hidden = torch.nn.functional.gelu(n @ gate_w.float().t(), approximate="tanh") * (n @ up_w.float().t())
    exact = hidden @ down_w.float().t()
    relative = lambda y: float((y.float() - exact).norm() / exact.norm())
    assert relative(got) < max(2.0 * relative(expected), 0.05), (relative(got), relative(expected))


@pytest.mark.parametrize("precision", ("fp8", "nvfp4"))
def test_refit_refreshes_the_plans_in_place(device, precision):
    """After a weight refit the calibrated plans must compute with the new weights although their packed operands
    are not module buffers: copying a fresh plan's ``refit_tensors`` into the live plan's (what the broadcast does)
    leaves every device pointer unchanged, and both the eager call and a graph captured BEFORE the refit then give
    the fresh plan's result bit for bit."""
    hidden, inter, tokens = 256, 512, 300
    quantizer = L.quantization_backends.get("cuda", request(device, bits_=4))
    def weights(seed):
        return tuple(make_weight(shape, seed + i, std=0.05).to(device=device, dtype=torch.bfloat16)
                     for i, shape in enumerate(((inter, hidden), (inter, hidden), (hidden, inter))))
    def build(seed):
        gate, up, down = weights(seed)
        return FusedMlpPlan(gate, up, down, gate_up_max=6.0, down_max=4.0, gate_up=precision, down=precision,
                            quantizer=quantizer, approximate="tanh")
    live, fresh = build(1), build(50)
    x = make_input((tokens, hidden), 7).to(device)
    before = live(x).clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(2):
            live(x)
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            captured = live(x)
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize()
    pointers = {name: tensor.data_ptr() for name, tensor in live.refit_tensors().items()}
    assert pointers and set(pointers) == set(fresh.refit_tensors())
    with torch.no_grad():
        for name, tensor in live.refit_tensors().items():
            tensor.copy_(fresh.refit_tensors()[name])
    assert {name: tensor.data_ptr() for name, tensor in live.refit_tensors().items()} == pointers
    want = fresh(x)
    after = live(x)
    assert torch.equal(after, want) and not torch.equal(after, before)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, want)


def test_bf16_outlier_channels_beside_the_nvfp4_mlp(device):
    """Hidden channels listed as outliers leave the NVFP4 path (their gate/up rows and down columns are packed as
    zeros) and are computed in bf16 beside it, as in the reference's ``MlpPlan._add_outliers``
    (policies/pi05/inference/mlp.py:119-131, 242-260).  The result is exactly the zeroed NVFP4 MLP plus the bf16 side
    path, and it is closer to the unquantised MLP than the plain NVFP4 plan when those channels carry huge values."""
    hidden, inter, tokens = 256, 512, 200
    quantizer = L.quantization_backends.get("cuda", request(device, bits_=4))
    gate = make_weight((inter, hidden), 1, std=0.05).to(device=device, dtype=torch.bfloat16)
    up = make_weight((inter, hidden), 2, std=0.05).to(device=device, dtype=torch.bfloat16)
    down = make_weight((hidden, inter), 3, std=0.05).to(device=device, dtype=torch.bfloat16)
    outliers = (5, 130, 131, 400)
    with torch.no_grad():
        gate[list(outliers)] *= 30                   # these hidden channels dwarf their neighbours' block scales
        up[list(outliers)] *= 30
    x = make_input((tokens, hidden), 9, outliers=False).to(device)
    exact = torch.nn.functional.gelu(x.float() @ gate.float().t(), approximate="tanh") * (x.float() @ up.float().t())
    hidden_peak = float(exact.abs().max())
    exact = exact @ down.float().t()
    kept = [c for c in range(inter) if c not in outliers]
    kept_peak = float((torch.nn.functional.gelu(x.float() @ gate.float()[kept].t(), approximate="tanh") * (x.float() @ up.float()[kept].t())).abs().max())
    common = dict(gate_up_max=float(x.abs().max()), gate_up="nvfp4", down="nvfp4", quantizer=quantizer, approximate="tanh")
    plain = FusedMlpPlan(gate, up, down, down_max=hidden_peak, **common)
    protected = FusedMlpPlan(gate, up, down, down_max=kept_peak, outliers=outliers, **common)
    got = protected(x).clone()
    # composition: the same plan without the side path on zeroed weights, plus the side path by hand
    index = torch.tensor(outliers, device=device)
    gate0, up0, down0 = gate.clone(), up.clone(), down.clone()
    gate0[index] = 0
    up0[index] = 0
    down0[:, index] = 0
    zeroed = FusedMlpPlan(gate0, up0, down0, down_max=kept_peak, **common)(x).clone()
    side = torch.nn.functional.gelu(x @ gate[index].t(), approximate="tanh") * (x @ up[index].t())
    assert torch.equal(got, zeroed.addmm_(side, down[:, index].t().contiguous()))
    error = lambda y: float((y.float() - exact).norm() / exact.norm())
    assert error(got) < 0.5 * error(plain(x)), (error(got), error(plain(x)))
    assert set(protected.refit_tensors()) >= {"side_gate_up", "side_down"}
    with pytest.raises(ValueError, match="exceed the MLP width"):
        FusedMlpPlan(gate, up, down, down_max=1.0, outliers=(inter,), **common)
    with pytest.raises(ValueError, match="require NVFP4"):
        FusedMlpPlan(gate, up, down, gate_up_max=1.0, down_max=1.0, gate_up="fp8", down="fp8", quantizer=quantizer, outliers=(1,))
