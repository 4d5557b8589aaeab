"""One-time weight conversion to the FP8 / NVFP4 bundle formats (not on the hot path).

These run once per checkpoint load on whatever device the weights live on, with plain tensor
operations, and produce exactly the buffers the reference's bundles hold:
  FP8    e4m3 [N, K] + fp32 scale () or [N]                 (embodiinfer/backend/torch/fp8.py:12-40, 76-96)
  NVFP4  packed e2m1 [N, K/2] + e4m3 [N, K/16] + fp32 ()    (embodiinfer/backend/torch/nvfp4.py:14-66)
The arithmetic (operation order, rounding points, tie handling) follows those functions so that
bundles made here and there are byte-identical.
"""

from __future__ import annotations

import math

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E2M1_THRESHOLDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
FP8_MAX = 448.0
_TINY = torch.finfo(torch.float32).tiny


def _e4m3() -> torch.dtype:
    dtype = getattr(torch, "float8_e4m3fn", None)
    if dtype is None:
        raise RuntimeError("this PyTorch build does not expose torch.float8_e4m3fn")
    return dtype


# ---- FP8 -------------------------------------------------------------------------------------------

def fp8_quantize_tensorwise(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """One fp32 scale for the whole matrix: amax/448 (1.0 for an all-zero matrix)."""
    values = weight.float()
    peak = values.abs().amax()
    scale = torch.where(peak > 0, peak / FP8_MAX, torch.ones_like(peak))
    return (values / scale).clamp(-FP8_MAX, FP8_MAX).to(_e4m3()), scale.float()


def fp8_quantize_channelwise(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """One fp32 scale per output row (the pre-Blackwell layout; kept so such bundles still load)."""
    values = weight.float()
    peak = values.abs().amax(dim=1)
    scale = torch.where(peak > 0, peak / FP8_MAX, torch.ones_like(peak))
    return (values / scale[:, None]).clamp(-FP8_MAX, FP8_MAX).to(_e4m3()), scale


def fp8_quantize_weight(
    weight: torch.Tensor, *, backend: str = "auto", scaling_scheme: str = "auto"
) -> tuple[torch.Tensor, torch.Tensor]:
    """``auto`` means tensorwise on a Blackwell CUDA device with a native-capable backend, else channelwise."""
    if scaling_scheme == "auto":
        blackwell = (
            weight.is_cuda and backend in {"auto", "native"} and torch.cuda.get_device_capability(weight.device)[0] >= 10
        )
        scaling_scheme = "tensorwise" if blackwell else "channelwise"
    if scaling_scheme == "tensorwise":
        return fp8_quantize_tensorwise(weight)
    return fp8_quantize_channelwise(weight)


def fp8_dequantize_weight(weight: torch.Tensor, weight_scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    scale = weight_scale.to(dtype)
    return weight.to(dtype) * (scale if scale.ndim == 0 else scale[:, None])


# ---- NVFP4 -----------------------------------------------------------------------------------------

def nvfp4_thresholds(like: torch.Tensor) -> torch.Tensor:
    return like.new_tensor(E2M1_THRESHOLDS, dtype=torch.float32)


def nvfp4_quantize_weight(
    values: torch.Tensor, thresholds: torch.Tensor | None = None
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[R, K] -> (packed uint8 [R, K/2], e4m3 block scales [R, K/16], fp32 global scale).

    global = max(amax, tiny)/2688; block scale = e4m3(clamp(blockmax/6/global, tiny, 448));
    code magnitude = number of thresholds strictly below |x/(global*scale)| (ties go to the smaller
    magnitude, NaN from an all-zero block counts all seven); bit 3 = value < 0; even column in the
    low nibble.
    """
    if values.ndim != 2 or values.shape[1] % 16:
        raise ValueError("NVFP4 quantization expects [M, K] with K divisible by 16")
    rows, columns = values.shape
    if thresholds is None:
        thresholds = nvfp4_thresholds(values)
    grid = values.float().view(rows, columns // 16, 16)
    overall = grid.abs().amax().clamp_min(_TINY) / (FP8_MAX * 6.0)
    per_block = (grid.abs().amax(dim=-1) / 6.0 / overall).clamp(_TINY, FP8_MAX).to(_e4m3())
    scaled = (grid / (overall * per_block.float())[..., None]).clamp(-6.0, 6.0).view(rows, columns)
    codes = torch.bucketize(scaled.abs(), thresholds).to(torch.uint8) | ((scaled < 0).to(torch.uint8) << 3)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed.contiguous(), per_block.contiguous(), overall.float()


def nvfp4_dequantize_weight(
    packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor, dtype: torch.dtype
) -> torch.Tensor:
    rows, half = packed.shape
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), device=packed.device, dtype=torch.float32)
    nibbles = torch.stack((packed & 0x0F, packed >> 4), dim=-1).view(rows, half * 2)
    values = table[nibbles.long()].view(rows, -1, 16)
    values = values * block_scale.view(_e4m3()).float()[..., None] * global_scale
    return values.view(rows, half * 2).to(dtype)


def blocked_scales(scales: torch.Tensor) -> torch.Tensor:
    """Row-major [R, Kb] block scales -> the 128x4-tile order, zero padded, flat.

    Byte (r, c) moves to ((r//128)*ceil(Kb/4) + c//4)*512 + (r%32)*16 + ((r%128)//32)*4 + c%4.
    """
    rows, columns = scales.shape
    row_tiles, column_tiles = math.ceil(rows / 128), math.ceil(columns / 4)
    padded = torch.zeros((row_tiles * 128, column_tiles * 4), dtype=scales.dtype, device=scales.device)
    padded[:rows, :columns] = scales
    # [row tile, quarter(4), row in quarter(32), column tile, column in tile(4)] -> [rt, ct, 32, quarter, 4]
    tiles = padded.view(row_tiles, 4, 32, column_tiles, 4).permute(0, 3, 2, 1, 4)
    return tiles.reshape(-1).contiguous()
