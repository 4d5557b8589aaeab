"""The C-ABI shared object: loads, exports every symbol the header declares, rejects bad
arguments with its documented codes.  No kernel is launched here."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from embodiinfer_b200 import _native as N

HEADER = Path(__file__).resolve().parent.parent / "include" / "embodiinfer_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return re.findall(r"^\s*(?:int|int64_t)\s+(b2_\w+)\s*\(", text, flags=re.M)


def test_library_exports_every_declared_symbol():
    library = N.load()
    names = declared_functions()
    assert {"b2_abi_version", "b2_tensor_scale", "b2_fp8_quantize", "b2_nvfp4_quantize", "b2_geglu", "b2_linear"} <= set(names)
    for name in names:
        assert hasattr(library, name), f"{name} is declared in the header but not exported"
        assert name in N.SIGNATURES, f"{name} has no ctypes signature"
    assert library.b2_abi_version() == N.ABI_VERSION


def test_header_constants_match_python_mirror():
    text = HEADER.read_text()
    values = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"#define\s+(B2_\w+)\s+\(?(-?\w+)\)?\s", text) if re.fullmatch(r"-?(0x)?[0-9a-fA-F]+", m.group(2))}
    for name in ("SPEC_T", "SPEC_C", "SCALAR_RCP", "DIVISOR_BF16", "CLAMP_TINY", "GEGLU_TRUE_DIV", "KIND_FP8", "KIND_NVFP4",
                 "EPI_LINEAR", "EPI_GEGLU", "OUT_BF16", "OUT_FP8", "OUT_NVFP4", "LINEAR_ROUND_SCALE_BF16", "LINEAR_PAIRED_GATE_UP_SCALES",
                 "LINEAR_STREAM_TOKENS",
                 "SCALE_SCRATCH_BYTES", "ABI_VERSION", "E_INVALID", "E_UNSUPPORTED", "E_DRIVER", "E_TOO_LARGE"):
        assert values[f"B2_{name}"] == getattr(N, name), name


def test_linear_desc_layout_matches_header():
    text = HEADER.read_text()
    body = re.search(r"typedef struct b2_linear_desc \{(.*?)\} b2_linear_desc;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = re.findall(r"(?:const\s+)?(?:int32_t|int64_t|void\*|b2_rope_desc\*)\s+(\w+);", body)
    assert fields == [name for name, _ in N.LinearDesc._fields_]


def test_argument_rejection_without_a_gpu():
    library = N.load()
    assert library.b2_fp8_quantize(None, None, None, 0, 0, None) == N.E_INVALID
    assert library.b2_tensor_scale(None, 16, 448.0, 0, None, None, None) == N.E_INVALID
    assert library.b2_nvfp4_quantize(None, None, None, None, None, 4, 64, 0, None) == N.E_INVALID
    assert library.b2_geglu(None, None, None, None, None, None, 4, 64, 64, 8, None, 0, None) == N.E_INVALID
    assert library.b2_linear(None, None) == N.E_INVALID
    fake = ctypes.c_void_p(4096)   # aligned, never dereferenced: checks happen before any launch
    assert library.b2_nvfp4_quantize(fake, fake, None, None, fake, 4, 24, 0, None) == N.E_UNSUPPORTED
    assert library.b2_geglu(fake, fake, fake, None, None, fake, 4, 64, 32, 8, fake, 0, None) == N.E_INVALID
    assert library.b2_geglu(fake, fake, fake, None, None, fake, 4, 64, 64, 5, fake, 0, None) == N.E_UNSUPPORTED
    assert library.b2_rope_split(None, None, None, None, None, None, 1, 4, 8, 1, 256, 0, 4, 0, None) == N.E_INVALID
    assert library.b2_rope_split(fake, fake, fake, fake, fake, fake, 1, 4, 8, 1, 24, 0, 4, 0, None) == N.E_UNSUPPORTED   # head_dim % 16
    assert library.b2_rope_split(fake, fake, fake, fake, fake, fake, 1, 4, 8, 1, 256, 0, 3, 0, None) == N.E_INVALID      # capacity < tokens
    assert library.b2_norm_quant(None, None) == N.E_INVALID
    norm = N.NormDesc(input=4096, output=4096, scale=4096, global_scale=4096, rows=6, columns=64, tokens=3, bits=8)
    norm.columns = 48
    assert library.b2_norm_quant(ctypes.byref(norm), None) == N.E_UNSUPPORTED  # width % 64
    norm.columns = 16384
    assert library.b2_norm_quant(ctypes.byref(norm), None) == N.E_TOO_LARGE
    norm.columns, norm.tokens = 64, 4
    assert library.b2_norm_quant(ctypes.byref(norm), None) == N.E_INVALID      # rows % tokens
    norm.tokens, norm.bits = 3, 4
    assert library.b2_norm_quant(ctypes.byref(norm), None) == N.E_INVALID      # NVFP4 without the tiled scale buffer
    norm.bits, norm.scale = 8, None
    assert library.b2_norm_quant(ctypes.byref(norm), None) == N.E_INVALID      # neither scale nor modulation
    desc = N.LinearDesc(kind=7, tokens=1, features=8, width=16)
    assert library.b2_linear(ctypes.byref(desc), None) == N.E_UNSUPPORTED
    desc = N.LinearDesc(kind=N.KIND_FP8, tokens=4, features=8, width=24, act=4096, weight=4096, act_scale=4096,
                        weight_scale=4096, out=4096)
    assert library.b2_linear(ctypes.byref(desc), None) == N.E_UNSUPPORTED      # K % 16
    plan = N.LinearDesc(kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=10, features=128, width=32768)
    assert library.b2_linear_workspace_bytes(ctypes.byref(plan)) > 0          # 2 tiles, 256 K stages: K would be split
    plan.tokens, plan.features = 8960, 16384
    assert library.b2_linear_workspace_bytes(ctypes.byref(plan)) == 0
    desc.width, desc.act = 32, 4100
    assert library.b2_linear(ctypes.byref(desc), None) == N.E_INVALID          # misaligned operand


def test_check_raises_like_the_reference_wrappers():
    N.check(0, "x")
    with pytest.raises(RuntimeError, match="failed with error -2"):
        N.check(-2, "b2_linear")
    with pytest.raises(RuntimeError, match="failed with error 700"):
        N.check(700, "b2_linear")
