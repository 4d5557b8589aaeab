"""Generate tests/golden/calibration_golden.npz by running the REFERENCE's own calibration code on CPU.

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_calibration_golden.py

Stored: a synthetic schema-2 calibration document (as JSON text), the layer records the unmodified
``_apply_calibration`` (embodiinfer/policies/pi05/inference/presets.py:114-163) selects from it, and the outputs of
the unmodified ``smoothed_norm_scale`` / ``smoothed_adarms`` (embodiinfer/policies/pi05/inference/mlp.py:40-60) and
of the gate/up weight folding expression (mlp.py:111-117) on seeded tensors.
"""

from __future__ import annotations

import json
import sys
import tempfile
from dataclasses import asdict
from pathlib import Path

import numpy as np
import torch

sys.dont_write_bytecode = True

from embodiinfer.policies.pi05.inference.config import Pi05OptimizationConfig  # noqa: E402
from embodiinfer.policies.pi05.inference.mlp import smoothed_adarms, smoothed_norm_scale  # noqa: E402
from embodiinfer.policies.pi05.inference.presets import _apply_calibration  # noqa: E402

OUT = Path(__file__).resolve().parent / "calibration_golden.npz"


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def synthetic_document() -> dict:
    generator = torch.Generator().manual_seed(77)
    smooth = lambda: [round(float(v), 4) for v in (torch.rand(64, generator=generator) * 3 + 0.25)]
    prefix = [{"gate_up": "nvfp4", "down": "nvfp4" if i % 5 else "bf16", "gate_up_max": 40.0 + i, "down_max": 200.0 + 3 * i,
               **({"smooth": smooth()} if i % 2 == 0 else {})} for i in range(18)]
    action = [{"gate_up": "fp8", "down": "fp8", "gate_up_max": 10.5 + i, "down_max": 90 + i} for i in range(18)]
    return {"schema_version": 2, "numerics": "openpi_rlinf", "activation": "gelu_pytorch_exact",
            "devices": {"spark": {"prefix": {"nvfp4": prefix}, "action": {"fp8": action}}},
            "checkpoint_sha256": "0" * 64}


def main() -> None:
    document = synthetic_document()
    config = Pi05OptimizationConfig(hardware="spark", numerics="openpi_rlinf", activation="gelu_pytorch_exact")
    with tempfile.TemporaryDirectory() as folder:
        path = Path(folder) / "calibration.json"
        path.write_text(json.dumps(document))
        resolved = _apply_calibration(config, {"prefix": "nvfp4", "action": "fp8"}, path)
    selected = {"prefix_layers": [asdict(layer) for layer in resolved.prefix_layers],
                "action_layers": [asdict(layer) for layer in resolved.action_layers],
                "checkpoint_sha256": resolved.checkpoint_sha256}
    generator = torch.Generator().manual_seed(78)
    width, inter = 64, 96
    norm_weight = (torch.randn(width, generator=generator) * 0.3).to(torch.bfloat16)
    smooth = torch.rand(width, generator=generator) * 3 + 0.25
    ada_weight = (torch.randn(3 * width, 48, generator=generator) * 0.2).to(torch.bfloat16)
    ada_bias = (torch.randn(3 * width, generator=generator) * 0.2).to(torch.bfloat16)
    gate = (torch.randn(inter, width, generator=generator) * 0.05).to(torch.bfloat16)
    folded_weight, folded_bias = smoothed_adarms(ada_weight, ada_bias, smooth)
    arrays = {
        "document": np.frombuffer(json.dumps(document).encode(), dtype=np.uint8),
        "selected": np.frombuffer(json.dumps(selected).encode(), dtype=np.uint8),
        "norm_weight": bits(norm_weight), "smooth": smooth.numpy().copy(),
        "norm_scale": smoothed_norm_scale(norm_weight, smooth).numpy().copy(),
        "ada_weight": bits(ada_weight), "ada_bias": bits(ada_bias),
        "ada_folded_weight": bits(folded_weight), "ada_folded_bias": bits(folded_bias),
        "gate": bits(gate), "gate_folded": bits((gate.float() * smooth).to(gate.dtype)),
    }
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
