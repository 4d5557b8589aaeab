"""Registry kernels ``fp8_native`` and ``nvfp4_native``: dynamic W8A8 / W4A4 Linear in three launches.

Drop-in for ``fp8.native_linear`` (embodiinfer/backend/torch/fp8.py:118-141) and
``nvfp4.native_linear`` (embodiinfer/backend/torch/nvfp4.py:96-123): same signature, same weight
bundle operands, same results as those functions produce on a CUDA device (tensor amax -> scale,
torch-route encoding arithmetic, scales applied the way each route does).  Where the reference
issues ~10 (FP8) or ~30 (NVFP4) elementwise launches around a library GEMM, this path issues
amax + encode + one fused tensor-core launch.
"""

from __future__ import annotations

import threading

import torch

from .. import _native as N
from .. import kernels as K
from .quantization import blocked_scale_bytes

_SUPPORTED_SM = (10, 0)   # the kernels are built for sm_100a only


class _Workspace:
    """Intermediate buffers for one (rows, K, device, stream); the bf16 output is fresh per call."""

    def __init__(self, rows: int, columns: int, bits: int, device: torch.device) -> None:
        self.scale = torch.zeros((), device=device, dtype=torch.float32)
        self.scratch = K.new_scale_scratch(device)
        if bits == 8:
            self.codes = torch.empty((rows, columns), device=device, dtype=torch.uint8)
            self.blocked = None
        else:
            self.codes = torch.empty((rows, columns // 2), device=device, dtype=torch.uint8)
            self.blocked = torch.zeros(blocked_scale_bytes(rows, columns), device=device, dtype=torch.uint8)


_workspaces: dict = {}
_workspaces_lock = threading.Lock()


def _workspace(rows: int, columns: int, bits: int, device: torch.device) -> _Workspace:
    key = (rows, columns, bits, device, torch.cuda.current_stream(device).cuda_stream)
    with _workspaces_lock:
        workspace = _workspaces.get(key)
        if workspace is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("Warm this shape once before CUDA Graph capture")
            workspace = _workspaces[key] = _Workspace(rows, columns, bits, device)
        return workspace


def release_workspaces() -> None:
    """Drop every cached intermediate buffer (call between models or after a refit)."""
    with _workspaces_lock:
        _workspaces.clear()


def _device_reason(inputs: torch.Tensor, method: str) -> str | None:
    if not inputs.is_cuda:
        return f"native {method} requires CUDA"
    capability = torch.cuda.get_device_capability(inputs.device)
    if capability != _SUPPORTED_SM:
        return f"native {method} is built for SM100 (B200) only, got SM{capability[0]}{capability[1]}"
    if not N.LIBRARY_PATH.exists():
        return f"{N.LIBRARY_PATH.name} is not built"
    return None


def fp8_native_capability(
    inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor
) -> tuple[bool, str | None]:
    """Hardware and alignment probe (fp8.py:99-115); no GEMM is launched."""
    reason = _device_reason(inputs, "FP8 W8A8")
    if reason is None and (weight.shape[1] % 16 or weight.shape[0] % 8):
        reason = "native FP8 W8A8 requires K divisible by 16 and N divisible by 8"
    if reason is None and inputs.dtype != torch.bfloat16:
        reason = "native FP8 W8A8 requires BF16 activations"
    return reason is None, reason


def nvfp4_native_capability(
    inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor
) -> tuple[bool, str | None]:
    """Hardware and alignment probe (nvfp4.py:73-93); ``weight`` is packed [N, K/2]."""
    reason = _device_reason(inputs, "NVFP4")
    if reason is None and ((weight.shape[1] * 2) % 64 or weight.shape[0] % 8):
        reason = "native NVFP4 requires K divisible by 64 and N divisible by 8"
    if reason is None and inputs.dtype != torch.bfloat16:
        reason = "native NVFP4 requires BF16 activations"
    return reason is None, reason


def no_fallback_capability(
    inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor
) -> tuple[bool, str | None]:
    return False, "this build has no CPU or weight-only fallback; use backend='native' on a B200"


def no_fallback_linear(inputs, weight, weight_scale, bias=None, **metadata):
    raise RuntimeError("this build has no CPU or weight-only fallback; use backend='native' on a B200")


def _rows(inputs: torch.Tensor, width: int) -> torch.Tensor:
    if inputs.dtype != torch.bfloat16:
        raise RuntimeError("native quantised Linear requires BF16 activations")
    return inputs.reshape(-1, width).contiguous()


def fp8_native_linear(
    inputs: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None
) -> torch.Tensor:
    """Dynamic per-tensor W8A8: ``bf16(scaled_mm(q(x), W^T, s_x, s_w)) + bias`` (fp8.py:118-141)."""
    if weight_scale.ndim != 0:
        raise RuntimeError(
            "SM100+ FP8 native dispatch requires tensorwise weights; load and quantize on CUDA "
            "or set scaling_scheme='tensorwise'"
        )
    features, width = weight.shape
    rows = _rows(inputs, width)
    tokens = rows.shape[0]
    device = rows.device
    ws = _workspace(tokens, width, 8, device)
    # fp8.py:70-72 as ATen evaluates it on CUDA: amax * fp32(1/448); bf16 quotient with a bf16 divisor.
    K.tensor_scale(rows, 448.0, N.SCALAR_RCP, ws.scratch, ws.scale)
    K.fp8_quantize(rows, ws.codes, ws.scale, N.SPEC_T | N.DIVISOR_BF16)
    output = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(
        kind=N.KIND_FP8, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features, width=width,
        act=ws.codes, act_scale=ws.scale, weight=weight, weight_scale=weight_scale.float(), out=output,
        bias=None if bias is None else bias.to(torch.bfloat16),
    )
    return output.reshape(*inputs.shape[:-1], features)


def nvfp4_native_linear(
    inputs: torch.Tensor,
    weight: torch.Tensor,
    weight_scale: torch.Tensor,
    bias: torch.Tensor | None = None,
    *,
    weight_global_scale: torch.Tensor,
    weight_scale_blocked: torch.Tensor,
    quantization_thresholds: torch.Tensor | None = None,
) -> torch.Tensor:
    """Dynamic W4A4: ``bf16(scaled_mm(...)) * bf16(g_x * g_w) + bias`` (nvfp4.py:96-123).

    ``quantization_thresholds`` is accepted for signature compatibility; the e2m1 decision
    boundaries are fixed constants of the encoder.
    """
    features, width = weight.shape[0], weight.shape[1] * 2
    rows = _rows(inputs, width)
    tokens = rows.shape[0]
    device = rows.device
    ws = _workspace(tokens, width, 4, device)
    # nvfp4.py:38-44 as ATen evaluates it on CUDA (python-scalar divisions become reciprocal multiplies).
    K.tensor_scale(rows, 448.0 * 6.0, N.SCALAR_RCP | N.CLAMP_TINY, ws.scratch, ws.scale)
    K.nvfp4_quantize(rows, ws.codes, None, ws.blocked, ws.scale, N.SPEC_T | N.SCALAR_RCP)
    output = torch.empty((tokens, features), device=device, dtype=torch.bfloat16)
    K.linear(
        kind=N.KIND_NVFP4, epilogue=N.EPI_LINEAR, out_format=N.OUT_BF16, tokens=tokens, features=features,
        width=width, act=ws.codes, act_scales=ws.blocked, act_scale=ws.scale, weight=weight,
        weight_scales=weight_scale_blocked, weight_scale=weight_global_scale.float(), out=output,
        bias=None if bias is None else bias.to(torch.bfloat16), flags=N.LINEAR_ROUND_SCALE_BF16,
    )
    return output.reshape(*inputs.shape[:-1], features)
