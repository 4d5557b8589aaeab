"""Host-side registries and configs: names, laziness, support checks, error behaviour.
Follows the reference's own registry tests (tests/test_operator_registry.py:31-91)."""

from __future__ import annotations

import sys

import pytest
import torch

from embodiinfer_b200 import layers as L
from embodiinfer_b200.layers import linear as LL
from embodiinfer_b200.layers.registry import BackendRegistry, OperatorCapabilities, OperatorRequest


def test_lazy_names_do_not_import_backends():
    for name in list(sys.modules):
        if name.startswith("embodiinfer_b200.backend."):
            del sys.modules[name]
    assert L.quantization_backends.available() == ("cuda", "native")
    assert L.projection_backends.available() == ("cuda", "native")
    assert L.gelu_mul_backends.available() == ("cuda", "native")
    assert not any(name.startswith("embodiinfer_b200.backend.quant") for name in sys.modules)


def test_unsupported_requests_fail_before_construction():
    built = []

    class Backend:
        capabilities = OperatorCapabilities(("cuda",), (torch.bfloat16,), "x", rank=2, width_multiple=64, bits=(4, 8))

        def __init__(self):
            built.append(self)

    registry = BackendRegistry("demo")
    registry.register("demo", Backend)
    with pytest.raises(ValueError, match="does not support cpu"):
        registry.get("demo", OperatorRequest(torch.device("cpu"), torch.bfloat16))
    with pytest.raises(ValueError, match="Unknown demo backend"):
        registry.get("other", OperatorRequest(torch.device("cpu"), torch.bfloat16))
    with pytest.raises(ValueError, match="already registered"):
        registry.register("demo", Backend)
    with pytest.raises(ValueError, match="Backend names"):
        registry.register(" padded", Backend)
    assert not built

    class CpuBackend:
        capabilities = OperatorCapabilities(("cpu",), (torch.bfloat16,), "x", rank=2, width_multiple=64, bits=(8,), cuda_graph=False)

    registry.register("cpu", CpuBackend)
    cpu = torch.device("cpu")
    with pytest.raises(ValueError, match="3-bit"):
        registry.get("cpu", OperatorRequest(cpu, torch.bfloat16, bits=3))
    with pytest.raises(ValueError, match="rank 2"):
        registry.get("cpu", OperatorRequest(cpu, torch.bfloat16, shape=(2, 3, 64)))
    with pytest.raises(ValueError, match="divisible by 64"):
        registry.get("cpu", OperatorRequest(cpu, torch.bfloat16, shape=(2, 65)))
    with pytest.raises(ValueError, match="CUDA Graph"):
        registry.get("cpu", OperatorRequest(cpu, torch.bfloat16, cuda_graph=True))
    with pytest.raises(ValueError, match="positive integer"):
        OperatorRequest(cpu, torch.bfloat16, shape=(0, 64))
    assert isinstance(registry.get("cpu", OperatorRequest(cpu, torch.bfloat16, shape=(2, 64), bits=8)), CpuBackend)

    class Undeclared:
        pass

    registry.register("undeclared", Undeclared)
    with pytest.raises(TypeError, match="must declare OperatorCapabilities"):
        registry.get("undeclared", OperatorRequest(cpu, torch.bfloat16))


def test_cuda_backends_reject_cpu_requests():
    request = OperatorRequest(torch.device("cpu"), torch.bfloat16, shape=(8, 64), bits=8)
    for registry in (L.quantization_backends, L.gelu_mul_backends, L.projection_backends):
        with pytest.raises(ValueError, match="does not support cpu"):
            registry.get("cuda", request)


def test_config_parsing():
    assert L.parse_quantization_config(None) is None
    assert L.parse_quantization_config("fp8") == L.FP8Config()
    assert L.parse_quantization_config("NVFP4") == L.NVFP4Config()
    config = L.parse_quantization_config({"method": "fp8", "backend": "native", "scaling_scheme": "tensorwise", "ignored_layers": ["*.o_proj"]})
    assert config == L.FP8Config(backend="native", scaling_scheme="tensorwise", ignored_layers=("*.o_proj",))
    assert config.is_ignored("layers.0.o_proj") and not config.is_ignored("layers.0.q_proj")
    assert L.parse_quantization_config({"quant_method": "nvfp4", "backend": "native"}) == L.NVFP4Config(backend="native")
    with pytest.raises(ValueError, match="unsupported quantization method"):
        L.parse_quantization_config("int4")
    with pytest.raises(TypeError, match="unknown FP8 config fields"):
        L.parse_fp8_config({"method": "fp8", "bogus": 1})
    with pytest.raises(TypeError, match="ignored_layers"):
        L.parse_nvfp4_config({"method": "nvfp4", "ignored_layers": "abc"})
    with pytest.raises(ValueError, match="activation_scheme"):
        L.FP8Config(activation_scheme="static")
    with pytest.raises(ValueError, match="unsupported NVFP4 backend"):
        L.NVFP4Config(backend="triton")
    with pytest.raises(ValueError, match="scaling_scheme"):
        L.FP8Config(scaling_scheme="blockwise")


def test_linear_backend_resolution_on_cpu_inputs():
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    w = torch.zeros(16, 64, dtype=torch.uint8)
    scale = torch.ones(())
    # CPU inputs resolve to "torch" like the reference (layers/linear.py:302-303) ...
    assert L.resolve_linear_backend("fp8", "auto", x, w, scale) == "torch"
    assert L.resolve_linear_backend("nvfp4", "native", x, w, scale) == "torch"
    # ... but this build ships no CPU fallback behind that name.
    with pytest.raises(RuntimeError, match="no CPU or weight-only fallback"):
        L.get_linear_backend("fp8_torch")(x, w, scale)
    with pytest.raises(ValueError, match="unsupported quantization method"):
        L.resolve_linear_backend("int8", "auto", x, w, scale)
    with pytest.raises(ValueError, match="unknown linear backend"):
        L.get_linear_backend("fp8_missing")
    with pytest.raises(ValueError, match="already registered"):
        L.register_linear("fp8_native", lambda *a, **k: None)


def test_native_capability_reasons_on_cpu():
    from embodiinfer_b200.backend import linear as BL

    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    ok, reason = BL.fp8_native_capability(x, torch.zeros(16, 64, dtype=torch.uint8), torch.ones(()))
    assert not ok and "requires CUDA" in reason
    ok, reason = BL.nvfp4_native_capability(x, torch.zeros(16, 32, dtype=torch.uint8), torch.ones(()))
    assert not ok and "requires CUDA" in reason


def test_register_custom_linear_and_explicit_backend_error(monkeypatch):
    calls = []

    def kernel(inputs, weight, weight_scale, bias=None, **metadata):
        calls.append(metadata)
        return inputs

    monkeypatch.setitem(LL._REGISTRY, "fp8_custom", (kernel, lambda *a: (False, "custom is off")))
    x = torch.zeros(2, 64, dtype=torch.bfloat16)

    class FakeCuda(torch.Tensor):
        is_cuda = True

    fake = x.as_subclass(FakeCuda)
    with pytest.raises(RuntimeError, match="custom is off"):
        L.resolve_linear_backend("fp8", "custom", fake, x, x)
