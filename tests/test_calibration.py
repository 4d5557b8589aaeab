"""The calibration loader, the layer record and the SmoothQuant folding against outputs of the reference's own
functions on CPU (tests/golden/make_calibration_golden.py), plus the validation errors."""

from __future__ import annotations

import copy
import json
from dataclasses import asdict
from pathlib import Path

import numpy as np
import pytest
import torch

from embodiinfer_b200 import calibration as C


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(Path(__file__).parent / "golden" / "calibration_golden.npz"))


def bf16(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(array.view(np.int16).copy()).view(torch.bfloat16)


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).numpy().view(np.uint16)


def test_loader_selects_what_the_reference_selects(golden, tmp_path):
    document = json.loads(golden["document"].tobytes().decode())
    expected = json.loads(golden["selected"].tobytes().decode())
    path = tmp_path / "calibration.json"
    path.write_text(json.dumps(document))
    for source in (path, str(path), document):
        loaded = C.load_calibration(source, hardware="spark", formats={"prefix": "nvfp4", "action": "fp8"})
        assert json.loads(json.dumps([asdict(layer) for layer in loaded.prefix_layers])) == expected["prefix_layers"]
        assert json.loads(json.dumps([asdict(layer) for layer in loaded.action_layers])) == expected["action_layers"]
        assert loaded.checkpoint_sha256 == expected["checkpoint_sha256"]
    only_action = C.load_calibration(document, hardware="spark", formats={"prefix": "bf16", "action": "fp8"})
    assert only_action.prefix_layers is None and len(only_action.action_layers) == 18


def test_loader_errors(golden):
    document = json.loads(golden["document"].tobytes().decode())
    formats = {"prefix": "nvfp4", "action": "fp8"}
    for key, value in (("schema_version", 1), ("schema_version", 2.0), ("numerics", "other"), ("activation", "tanh")):
        broken = {**document, key: value}
        with pytest.raises(ValueError, match="schema 2"):
            C.load_calibration(broken, hardware="spark", formats=formats)
    with pytest.raises(ValueError, match="no ranges for b200"):
        C.load_calibration(document, hardware="b200", formats=formats)
    with pytest.raises(ValueError, match="18 action MLP layer ranges for nvfp4"):
        C.load_calibration(document, hardware="spark", formats={"action": "nvfp4"})
    short = copy.deepcopy(document)
    short["devices"]["spark"]["prefix"]["nvfp4"].pop()
    with pytest.raises(ValueError, match="18 prefix MLP layer ranges"):
        C.load_calibration(short, hardware="spark", formats=formats)
    mixed = copy.deepcopy(document)
    mixed["devices"]["spark"]["action"]["fp8"][3]["down"] = "nvfp4"
    with pytest.raises(ValueError, match="must select fp8 with optional BF16 protection"):
        C.load_calibration(mixed, hardware="spark", formats=formats)
    unsigned = {key: value for key, value in document.items() if key != "checkpoint_sha256"}
    with pytest.raises(ValueError, match="checkpoint SHA256"):
        C.load_calibration(unsigned, hardware="spark", formats=formats)


def test_layer_record_validation():
    good = C.MlpLayerPrecision("nvfp4", "nvfp4", 3.0, 4, smooth=[1.0, 2.0], outliers=[5, 1])
    assert good.smooth == (1.0, 2.0) and good.outliers == (5, 1)
    cases = [
        (dict(gate_up="int8"), "MLP precision"),
        (dict(gate_up_max=0.0), "maxima"), (dict(down_max=float("inf")), "maxima"), (dict(gate_up_max=True), "maxima"),
        (dict(gate_up="fp8", smooth=[]), "SmoothQuant scales must be finite"),
        (dict(gate_up="fp8", smooth=[1.0, -1.0]), "SmoothQuant scales must be finite"),
        (dict(gate_up="bf16", smooth=[1.0]), "apply to quantized"),
        (dict(gate_up="nvfp4", outliers=[]), "distinct non-negative"), (dict(gate_up="nvfp4", outliers=[1, 1]), "distinct"),
        (dict(gate_up="nvfp4", outliers=[-1]), "distinct"), (dict(gate_up="fp8", outliers=[1]), "require NVFP4"),
    ]
    for arguments, message in cases:
        with pytest.raises(ValueError, match=message):
            C.MlpLayerPrecision(**arguments)


def test_smoothquant_folding_matches_the_reference(golden):
    smooth = torch.from_numpy(golden["smooth"])
    assert np.array_equal(C.smoothed_norm_scale(bf16(golden["norm_weight"]), smooth).numpy(), golden["norm_scale"])
    weight, bias = C.smoothed_adarms(bf16(golden["ada_weight"]), bf16(golden["ada_bias"]), smooth)
    assert np.array_equal(bits(weight), golden["ada_folded_weight"]) and np.array_equal(bits(bias), golden["ada_folded_bias"])
    gate = bf16(golden["gate"])
    layer = C.MlpLayerPrecision("fp8", "fp8", 1.0, 1.0, smooth=[float(value) for value in golden["smooth"]])
    folded_gate, folded_up = C.smoothed_projection_weights(gate, gate.clone(), layer)
    assert np.array_equal(bits(folded_gate), golden["gate_folded"]) and torch.equal(folded_gate, folded_up)
    plain = C.MlpLayerPrecision("fp8", "fp8", 1.0, 1.0)
    assert C.smoothed_projection_weights(gate, gate, plain)[0] is gate
    with pytest.raises(ValueError, match="input width"):
        C.smoothed_projection_weights(gate[:, :32], gate[:, :32], layer)


def test_folding_leaves_the_mlp_input_product_unchanged():
    """(x / s) @ (W * s)^T == x @ W^T up to rounding: the property SmoothQuant rests on."""
    generator = torch.Generator().manual_seed(5)
    x, w = torch.randn(7, 64, generator=generator), torch.randn(96, 64, generator=generator)
    s = torch.rand(64, generator=generator) * 3 + 0.25
    assert torch.allclose((x / s) @ (w * s).t(), x @ w.t(), atol=1e-4)
    norm_weight = torch.randn(64, generator=generator) * 0.3
    assert torch.allclose(1 + C.smoothed_norm_scale(norm_weight, s), (1 + norm_weight) / s, atol=1e-6)


def test_plan_builder_rejects_layouts_without_a_gpu():
    gate = torch.zeros((96, 64), dtype=torch.bfloat16)
    down = torch.zeros((64, 96), dtype=torch.bfloat16)
    layer = C.MlpLayerPrecision("nvfp4", "nvfp4", 1.0, 1.0, outliers=[96])
    with pytest.raises(ValueError, match="Outlier channels exceed the MLP width"):
        C.fused_mlp_from_layer(gate, gate, down, layer, quantizer=None)
    with pytest.raises(ValueError, match="dimensions do not match"):
        C.fused_mlp_from_layer(gate, gate, gate, C.MlpLayerPrecision("fp8", "fp8"), quantizer=None)
    with pytest.raises(ValueError, match="BF16 projection weights"):
        C.fused_mlp_from_layer(gate.float(), gate.float(), down.float(), C.MlpLayerPrecision("fp8", "fp8"), quantizer=None)


def test_presets_resolve_like_the_reference():
    """``resolve_preset`` for the B200 launch profile: the reference's preset names, checks and messages
    (policies/pi05/inference/presets.py:27-112), ranges from a schema-2 document."""
    row = dict(gate_up="nvfp4", down="nvfp4", gate_up_max=3.0, down_max=40.0)
    document = {"schema_version": 2, "numerics": "openpi_rlinf", "activation": "gelu_pytorch_exact", "checkpoint_sha256": "ab" * 32,
                "devices": {"b200": {"prefix": {"nvfp4": [dict(row, outliers=[7]) if i == 3 else row for i in range(18)]},
                                     "action": {"fp8": [dict(gate_up="fp8", down="fp8", gate_up_max=2.0, down_max=9.0)] * 18}}}}
    recipe = C.resolve_preset("b200", "nvfp4-fp8", calibration=document)
    assert (recipe.prefix, recipe.action, recipe.fused_mlp, recipe.checkpoint_sha256) == ("nvfp4", "fp8", True, "ab" * 32)
    assert len(recipe.prefix_layers) == len(recipe.action_layers) == 18 and recipe.prefix_layers[3].outliers == (7,)
    assert recipe.operators["norm_quant"] == "b200" and recipe.has_quantized_mlp
    assert C.resolve_preset("b200", "strict", calibration=None) == C.Recipe(hardware="b200")
    assert not C.resolve_preset("b200", "bf16", calibration=None).has_quantized_mlp
    with pytest.raises(ValueError, match="Unknown Pi05 device 'thor'"):
        C.resolve_preset("thor", "fp8-fp8", calibration=document)
    with pytest.raises(ValueError, match="strict BF16 preset does not use calibration"):
        C.resolve_preset("b200", "strict", calibration=document)
    with pytest.raises(ValueError, match="Integer MLP presets require Orin"):
        C.resolve_preset("b200", "w4a16", calibration=document)
    with pytest.raises(ValueError, match="prefix-action format pair"):
        C.resolve_preset("b200", "int8-int8", calibration=document)
    with pytest.raises(ValueError, match="requires 18 action MLP layer ranges for nvfp4"):
        C.resolve_preset("b200", "nvfp4-nvfp4", calibration=document)
    with pytest.raises(ValueError, match="no ranges for b200"):
        C.resolve_preset("b200", "fp8-fp8", calibration=None)
