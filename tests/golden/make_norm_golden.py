"""Generate tests/golden/norm_golden.npz by running the REFERENCE's own CPU normalisation.

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_norm_golden.py

Every array is a seeded input or the output of the unmodified
``TorchRMSNorm().plan(...).normalize / residual_normalize``
(embodiinfer/backend/torch/normalization.py:49-103).  ``*_inverse`` is torch's own
``rsqrt(inputs.float().square().mean(-1) + eps)`` on CPU, recomputed here with the same expression, so a
restatement of the affine arithmetic can be fed the identical factor.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

sys.dont_write_bytecode = True

from embodiinfer.backend.torch.normalization import TorchRMSNorm  # noqa: E402

OUT = Path(__file__).resolve().parent / "norm_golden.npz"

CASES = {  # name -> (batch, tokens, columns, seed, adaptive, with update, with update gate)
    "plain": (2, 5, 64, 301, False, False, False),
    "wide": (1, 7, 2048, 302, False, False, False),
    "residual": (2, 3, 1024, 303, False, True, False),
    "adaptive": (3, 4, 1024, 304, True, False, False),
    "adaptive_gated": (2, 10, 1024, 305, True, True, True),
    "odd_width": (2, 3, 1152, 306, False, True, False),
}


def bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main() -> None:
    arrays: dict[str, np.ndarray] = {}
    for name, (batch, tokens, columns, seed, adaptive, with_update, with_gate) in CASES.items():
        generator = torch.Generator().manual_seed(seed)
        inputs = (torch.randn((batch, tokens, columns), generator=generator) * 3).to(torch.bfloat16)
        inputs[0, 0, :16] = 0
        update = torch.randn((batch, tokens, columns), generator=generator).to(torch.bfloat16) if with_update else None
        gate = torch.randn((batch, 1, columns), generator=generator).to(torch.bfloat16) if with_gate else None
        scale = torch.randn((columns,), generator=generator) * 0.2
        modulation = torch.randn((batch, 3 * columns), generator=generator) * 0.3
        plan = TorchRMSNorm().plan(inputs, adaptive=adaptive)
        affine = {"modulation": modulation} if adaptive else {"scale": scale}
        if with_update:
            residual, normalized, next_gate = plan.residual_normalize(inputs, update, gate, **affine)
        else:
            normalized, next_gate = plan.normalize(inputs, **affine)
            residual = inputs
        inverse = torch.rsqrt(residual.float().square().mean(dim=-1, keepdim=True) + plan.eps)
        arrays[f"{name}_inputs"] = bits(inputs.reshape(-1, columns))
        arrays[f"{name}_tokens"] = np.int64(tokens)
        if with_update:
            arrays[f"{name}_update"] = bits(update.reshape(-1, columns))
        if with_gate:
            arrays[f"{name}_update_gate"] = bits(gate.reshape(-1, columns))
        arrays[f"{name}_scale" if not adaptive else f"{name}_modulation"] = (modulation if adaptive else scale).numpy().copy()
        arrays[f"{name}_inverse"] = inverse.reshape(-1).numpy().copy()
        arrays[f"{name}_residual"] = bits(residual.reshape(-1, columns))
        arrays[f"{name}_normalized"] = bits(normalized.reshape(-1, columns))
        if next_gate is not None:
            arrays[f"{name}_gate"] = bits(next_gate.reshape(-1, columns))
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes, {len(arrays)} arrays)")


if __name__ == "__main__":
    main()
