"""Register the B200 kernels in a running EmbodiInfer process (no change to EmbodiInfer's sources).

    import embodiinfer_b200.integration as b200
    b200.register_into_reference()            # once, at start-up, before policies are built

What it does, through the reference's own registries:

* plan route: registers this package's backends under the name ``"b200"`` in ``quantization_backends``,
  ``projection_backends``, ``gelu_mul_backends`` and ``norm_quant_backends`` (embodiinfer/layers/quantization.py:84-101,
  layers/activation.py:71-74, layers/normalization.py:99-107) with the reference's public
  ``BackendRegistry.register``; a policy selects them through its operator configuration
  (``OperatorBackends(quantization="b200", gelu_mul="b200", projection="b200", norm_quant="b200")``).
  ``BackendRegistry.get`` checks ``isinstance(capabilities, OperatorCapabilities)`` against the reference's own
  class (layers/registry.py:126-128), so each class is registered as a subclass whose ``capabilities`` is rebuilt
  from that class with the same field values.
* registry route: ``QuantizedLinear.forward`` resolves ``"{method}_native"`` (layers/linear.py:288-314), and the
  configuration parser accepts no other back-end name, so ``fp8_native`` / ``nvfp4_native`` are pointed at this
  package's kernels and capability probes.  The reference offers no public call that replaces an entry, hence the
  assignment into its registry table.
"""

from __future__ import annotations

import dataclasses
import importlib


def _adapt(cls: type, reference_capabilities: type) -> type:
    """``cls`` with its capability declaration expressed in the reference's dataclass."""
    fields = {field.name for field in dataclasses.fields(reference_capabilities)}
    values = {name: value for name, value in dataclasses.asdict(cls.capabilities).items() if name in fields}
    return type(cls.__name__, (cls,), {"capabilities": reference_capabilities(**values), "__doc__": cls.__doc__})


def register_into_reference(name: str = "b200", *, replace_native_linear: bool = True, package: str = "embodiinfer") -> dict[str, list[str]]:
    """Returns what was registered, by registry.  Raises ``ValueError`` if ``name`` is taken (call it once)."""
    ref_registry = importlib.import_module(f"{package}.layers.registry")
    ref_quantization = importlib.import_module(f"{package}.layers.quantization")
    ref_activation = importlib.import_module(f"{package}.layers.activation")
    ref_normalization = importlib.import_module(f"{package}.layers.normalization")
    ref_linear = importlib.import_module(f"{package}.layers.linear")

    from .backend import linear as linear_kernels
    from .backend.activation import B200GeluMul
    from .backend.norm_quant import B200NormQuant
    from .backend.projection import B200ProjectionBackend
    from .backend.quantization import B200Quantizer

    capabilities = ref_registry.OperatorCapabilities
    done: dict[str, list[str]] = {}
    for registry, cls in ((ref_quantization.quantization_backends, B200Quantizer),
                          (ref_quantization.projection_backends, B200ProjectionBackend),
                          (ref_activation.gelu_mul_backends, B200GeluMul),
                          (ref_normalization.norm_quant_backends, B200NormQuant)):
        registry.register(name, _adapt(cls, capabilities))
        done.setdefault(registry.family, []).append(name)
    if replace_native_linear:
        ref_linear._REGISTRY["fp8_native"] = (linear_kernels.fp8_native_linear, linear_kernels.fp8_native_capability)
        ref_linear._REGISTRY["nvfp4_native"] = (linear_kernels.nvfp4_native_linear, linear_kernels.nvfp4_native_capability)
        done["linear"] = ["fp8_native", "nvfp4_native"]
    return done
