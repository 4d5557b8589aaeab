"""Registering the B200 back ends in the reference's own registries (embodiinfer_b200/integration.py), on CPU.

Needs the reference package: it is imported from ``baseline/_ref`` (``python baseline/install_reference.py
<checkout>``) and the test skips without it.  No kernel runs: what is checked is name resolution, the
capability objects' type (the reference's ``isinstance`` check) and the error behaviour of unsupported requests."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

REFERENCE = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


@pytest.fixture(scope="module")
def registered():
    if not (REFERENCE / "embodiinfer").exists():
        pytest.skip("baseline/_ref is not installed")
    sys.path.insert(0, str(REFERENCE))
    try:
        import embodiinfer  # noqa: F401
        from embodiinfer_b200.integration import register_into_reference

        yield register_into_reference()
    finally:
        sys.path.remove(str(REFERENCE))


def test_names_resolve_in_the_reference_registries(registered):
    from embodiinfer.layers import linear as ref_linear
    from embodiinfer.layers.activation import gelu_mul_backends
    from embodiinfer.layers.normalization import norm_quant_backends
    from embodiinfer.layers.quantization import projection_backends, quantization_backends
    from embodiinfer_b200.backend import linear as b200

    assert registered["linear"] == ["fp8_native", "nvfp4_native"]
    for registry in (quantization_backends, projection_backends, gelu_mul_backends, norm_quant_backends):
        assert "b200" in registry.available()
    assert ref_linear.get_linear_backend("fp8_native") is b200.fp8_native_linear
    assert ref_linear.get_linear_backend("nvfp4_native") is b200.nvfp4_native_linear
    # CPU inputs keep the reference's own torch route (layers/linear.py:300-301)
    x, w, s = torch.zeros(2, 64, dtype=torch.bfloat16), torch.zeros(16, 64, dtype=torch.uint8), torch.ones(())
    assert ref_linear.resolve_linear_backend("fp8", "auto", x, w, s) == "torch"
    with pytest.raises(ValueError, match="already registered"):
        from embodiinfer_b200.integration import register_into_reference
        register_into_reference()


def test_capability_checks_run_through_the_reference(registered):
    """``BackendRegistry.get`` of the reference accepts the classes (their capabilities are its own dataclass) and
    rejects unsupported requests with its own messages, before any construction."""
    from embodiinfer.layers.activation import gelu_mul_backends
    from embodiinfer.layers.normalization import norm_quant_backends
    from embodiinfer.layers.quantization import projection_backends, quantization_backends
    from embodiinfer.layers.registry import OperatorCapabilities, OperatorRequest

    for registry in (quantization_backends, projection_backends, gelu_mul_backends, norm_quant_backends):
        registry_class = registry._factories["b200"]
        assert isinstance(registry_class.capabilities, OperatorCapabilities)
        with pytest.raises(ValueError, match="does not support cpu"):
            registry.get("b200", OperatorRequest(torch.device("cpu"), torch.bfloat16))
    with pytest.raises(ValueError, match="does not support 3-bit"):
        quantization_backends.get("b200", OperatorRequest(torch.device("cuda"), torch.bfloat16, bits=3))
    with pytest.raises(ValueError, match="divisible by 64"):
        quantization_backends.get("b200", OperatorRequest(torch.device("cuda"), torch.bfloat16, shape=(8, 96), bits=8))
    if not torch.cuda.is_available():
        with pytest.raises(ValueError, match="requires an available CUDA device"):
            quantization_backends.get("b200", OperatorRequest(torch.device("cuda"), torch.bfloat16, shape=(8, 128), bits=8))
    # the arithmetic contracts the reference's caller compares (operators.py:181-191)
    assert quantization_backends._factories["b200"].capabilities.arithmetic == "rounded_bf16_encoding"
    assert gelu_mul_backends._factories["b200"].capabilities.arithmetic == "torch_gelu_product_bf16_rounding"
    assert norm_quant_backends._factories["b200"].capabilities.arithmetic == "torch_rmsnorm_bf16_rounding"
