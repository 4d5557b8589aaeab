"""ctypes binding of ``libembodiinfer_b200.so`` (the C ABI declared in include/embodiinfer_b200.h).

There is no fallback: if the shared object is missing the import of any operator raises.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libembodiinfer_b200.so"

# Mirrors of the header's constants.
OK = 0
E_INVALID, E_UNSUPPORTED, E_DRIVER, E_TOO_LARGE = -1, -2, -3, -4
SPEC_T, SPEC_C, SCALAR_RCP, DIVISOR_BF16, CLAMP_TINY, GEGLU_TRUE_DIV = 0, 1, 2, 4, 8, 16
KIND_FP8, KIND_NVFP4 = 0, 1
EPI_LINEAR, EPI_GEGLU, EPI_GELU = 0, 1, 2
OUT_BF16, OUT_FP8, OUT_NVFP4 = 0, 1, 2
LINEAR_ROUND_SCALE_BF16 = 1
LINEAR_PAIRED_GATE_UP_SCALES = 4
LINEAR_STREAM_TOKENS = 8
LINEAR_SINGLE_CTA = 64
LINEAR_PAIRS = 128
LINEAR_CLUSTER = 256
NORM_RESIDUAL_EVICT_LAST = 1
SCALE_SCRATCH_BYTES = 8
STATIC_SCRATCH_BYTES = 16640
STATIC_SCALE_MAX_COUNT = 67108864
ABI_VERSION = 7

_ERRORS = {
    E_INVALID: "invalid argument (null, non-positive size or misaligned pointer)",
    E_UNSUPPORTED: "unsupported shape or mode",
    E_DRIVER: "tensor-map creation failed",
    E_TOO_LARGE: "size beyond the entry point's maximum",
}


class LinearDesc(ctypes.Structure):
    """``b2_linear_desc``."""

    _fields_ = [
        ("kind", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("out_format", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("features", ctypes.c_int32),
        ("width", ctypes.c_int32),
        ("feature_tile", ctypes.c_int32),
        ("gelu_lo", ctypes.c_int32),
        ("gelu_hi", ctypes.c_int32),
        ("act", ctypes.c_void_p),
        ("act_scales", ctypes.c_void_p),
        ("act_scale", ctypes.c_void_p),
        ("weight", ctypes.c_void_p),
        ("weight_scales", ctypes.c_void_p),
        ("weight_scale", ctypes.c_void_p),
        ("weight_scale_up", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p),
        ("gelu_table", ctypes.c_void_p),
        ("out_scale", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("out_scales", ctypes.c_void_p),
        ("out_blocked", ctypes.c_void_p),
        ("status", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64),
        ("rope", ctypes.c_void_p),
    ]


class RopeDesc(ctypes.Structure):
    """``b2_rope_desc``."""

    _fields_ = [(name, ctypes.c_void_p) for name in ("sine", "cosine", "q_out", "k_out", "v_out")] + \
               [("factor_batch_stride", ctypes.c_int64)] + \
               [(name, ctypes.c_int32) for name in ("batch", "tokens", "heads", "kv_heads", "head_dim", "kv_capacity", "kv_offset")]


class NormDesc(ctypes.Structure):
    """``b2_norm_desc``."""

    _fields_ = [(name, ctypes.c_void_p) for name in (
        "input", "update", "update_gate", "scale", "modulation", "mean", "global_scale", "residual", "output", "scales",
        "blocked", "gate", "inverse")] + [(name, ctypes.c_int32) for name in ("rows", "columns", "tokens", "bits", "flags")]


_P, _I, _I64, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

# name -> argtypes; every entry returns int.
SIGNATURES: dict[str, list] = {
    "b2_abi_version": [],
    "b2_tensor_scale": [_P, _I64, _F, _I, _P, _P, _P],
    "b2_tensor_scale_static": [_P, _I64, _F, _I, _P, _P],
    "b2_fp8_quantize": [_P, _P, _P, _I64, _I, _P],
    "b2_nvfp4_quantize": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "b2_geglu": [_P, _P, _P, _P, _P, _P, _I, _I, _I64, _I, _P, _I, _P],
    "b2_linear": [ctypes.POINTER(LinearDesc), _P],
    "b2_gelu_table_range": [_P, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)],
    "b2_linear_workspace_bytes": [ctypes.POINTER(LinearDesc)],
    "b2_norm_quant": [ctypes.POINTER(NormDesc), _P],
    "b2_layer_norm_quant": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _P],
    "b2_bhsd_quant": [_P, _P, _P, _P, _F, _I64, _I64, _I64, _I, _I, _I, _I, _I, _P],
    "b2_normalize_frames": [_P, _P, _I, _I, _P],
    "b2_frames_to_patches": [_P, _P, _I, _I, _I, _I, _P],
    "b2_resize_frames": [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "b2_rope_split": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I64, _I, _I, _P],
    "b2_attention": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "b2_attention_fp8": [_P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _P, _P],
    "b2_attention_nvfp4": [_P, _P, _P, _P, _P, _P, _F, _I, _I, _I, _I, _I, _P, _P],
}
RESULT_TYPES = {"b2_linear_workspace_bytes": ctypes.c_int64}

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load the shared object once and declare every entry point's signature."""
    global _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.exists():
                raise RuntimeError(
                    f"{LIBRARY_PATH} is missing: build it with `python -m embodiinfer_b200.build` "
                    "(there is no CPU or library fallback for this path)"
                )
            library = ctypes.CDLL(str(LIBRARY_PATH))
            for name, argtypes in SIGNATURES.items():
                function = getattr(library, name, None)
                if function is None:
                    raise RuntimeError(f"{LIBRARY_PATH} does not export {name}")
                function.argtypes = argtypes
                function.restype = RESULT_TYPES.get(name, ctypes.c_int)
            if library.b2_abi_version() != ABI_VERSION:
                raise RuntimeError("libembodiinfer_b200.so ABI version mismatch; rebuild it")
            _library = library
        return _library


def check(status: int, what: str) -> None:
    """Raise like the reference's wrappers do (backend/cuda/quantization.py:63-66)."""
    if status == 0:
        return
    detail = _ERRORS.get(status, f"CUDA error {status}" if status > 0 else "unknown error")
    raise RuntimeError(f"{what} failed with error {status}: {detail}")
