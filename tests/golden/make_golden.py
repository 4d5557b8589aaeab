"""Generate tests/golden/quant_golden.npz by running the REFERENCE's own CPU code.

Run in a container where the reference checkout is importable:

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

Every array stored here is either a seeded input or the output of an unmodified reference function:
  fp8._dynamic_fp8_activation_tensorwise   (embodiinfer/backend/torch/fp8.py:66-73)
  fp8._quantize_weight_per_tensor          (embodiinfer/backend/torch/fp8.py:32-40)
  TorchQuantizer().plan().quantize         (embodiinfer/backend/torch/quantization.py:43-57)
  nvfp4.quantize_weight / blocked_scales / dequantize_weight (embodiinfer/backend/torch/nvfp4.py:14-66)
  TorchGeluMul (separate GELU, product)    (embodiinfer/backend/torch/activation.py:55-60)
Large cases (the benchmark shapes) are stored as SHA-256 digests of inputs and outputs only.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

sys.dont_write_bytecode = True

from embodiinfer.backend.torch import fp8 as ref_fp8  # noqa: E402
from embodiinfer.backend.torch import nvfp4 as ref_nvfp4  # noqa: E402
from embodiinfer.backend.torch.quantization import TorchQuantizer  # noqa: E402

OUT = Path(__file__).resolve().parent / "quant_golden.npz"

SMALL_CASES = {  # name -> (shape, seed, multiplier)
    "a": ((37, 64), 101, 1.0),
    "b": ((130, 256), 102, 30.0),
    "c": ((16, 64), 103, 1e-3),
    "d": ((3, 16), 104, 1.0),
    "e": ((129, 64), 105, 4.0),
}
LARGE_CASES = {  # the benchmark shapes: digests only
    "cfg1_x": ((560, 2048), 1001, 1.0),
    "cfg2_x": ((560, 2048), 1002, 1.0),
    "cfg2_h": ((560, 16384), 1012, 1.0),
}


def make_input(shape, seed, multiplier):
    """bf16 activations ~N(0,1)*multiplier with 1% outliers x20, plus zero / signed-zero blocks."""
    generator = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=generator) * multiplier
    x = torch.where(torch.rand(shape, generator=generator) < 0.01, x * 20, x).to(torch.bfloat16)
    if len(shape) == 2 and shape[0] > 1 and shape[1] >= 32:
        x[0, :16] = 0
        x[1, 16:32] = torch.tensor([0.0, -0.0] * 8).to(torch.bfloat16)
    return x


def make_weight(shape, seed):
    generator = torch.Generator().manual_seed(seed + 5000)
    return torch.randn(shape, generator=generator) * 0.02


def bits(t):
    return t.contiguous().view(torch.uint16).numpy().copy()


def u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def reference_outputs(x):
    out = {}
    q, s = ref_fp8._dynamic_fp8_activation_tensorwise(x)
    out["fp8T_codes"], out["fp8T_scale"] = u8(q), np.float32(s.item())
    plan = TorchQuantizer().plan(x, 8).quantize(x)
    out["fp8C_dyn_codes"], out["fp8C_dyn_scale"] = u8(plan.output), np.float32(plan.scale.item())
    plan = TorchQuantizer().plan(x, 8, 0.0371).quantize(x)
    out["fp8C_static_codes"] = u8(plan.output)
    thresholds = ref_nvfp4.quantization_thresholds(x)
    packed, scales, g = ref_nvfp4.quantize_weight(x, thresholds)
    out["nv4T_packed"], out["nv4T_scales"], out["nv4T_global"] = packed.numpy().copy(), u8(scales), np.float32(g.item())
    out["nv4T_blocked"] = u8(ref_nvfp4.blocked_scales(scales))
    if x.numel() <= 4096:
        out["nv4T_dequant"] = ref_nvfp4.dequantize_weight(packed, scales, g, torch.float32).numpy().copy()
    return out


def main():
    store = {}
    for name, (shape, seed, multiplier) in SMALL_CASES.items():
        x = make_input(shape, seed, multiplier)
        store[f"{name}_x"] = bits(x)
        for key, value in reference_outputs(x).items():
            store[f"{name}_{key}"] = value
        w = make_weight(shape, seed)
        store[f"{name}_w"] = w.numpy().copy()
        q, s = ref_fp8._quantize_weight_per_tensor(w)
        store[f"{name}_wfp8_codes"], store[f"{name}_wfp8_scale"] = u8(q), np.float32(s.item())
        packed, scales, g = ref_nvfp4.quantize_weight(w, ref_nvfp4.quantization_thresholds(w))
        store[f"{name}_wnv4_packed"], store[f"{name}_wnv4_scales"] = packed.numpy().copy(), u8(scales)
        store[f"{name}_wnv4_global"] = np.float32(g.item())
        # GELU(gate) * up with separate bf16 roundings (activation.py:59)
        gate, up = x, make_input(shape, seed + 77, 1.0)
        store[f"{name}_up"] = bits(up)
        for approximate in ("tanh", "none"):
            hidden = torch.nn.functional.gelu(gate, approximate=approximate) * up
            store[f"{name}_hidden_{approximate}"] = bits(hidden)
    digests = []
    for name, (shape, seed, multiplier) in LARGE_CASES.items():
        x = make_input(shape, seed, multiplier)
        digests.append(f"{name}_x={hashlib.sha256(bits(x).tobytes()).hexdigest()}")
        for key, value in reference_outputs(x).items():
            if key.endswith("dequant"):
                continue
            digests.append(f"{name}_{key}={hashlib.sha256(np.asarray(value).tobytes()).hexdigest()}")
    store["digests"] = np.array(digests)
    codes = torch.arange(65536, dtype=torch.int32).to(torch.uint16).view(torch.bfloat16)
    for approximate in ("tanh", "none"):
        table = torch.nn.functional.gelu(codes, approximate=approximate).view(torch.uint16).numpy()
        store[f"gelu_table_{approximate}_sha256"] = np.array(hashlib.sha256(table.tobytes()).hexdigest())
    np.savez_compressed(OUT, **store)
    print(OUT, OUT.stat().st_size, "bytes", len(store), "arrays")


if __name__ == "__main__":
    main()
