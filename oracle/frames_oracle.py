"""CPU oracle for the camera-frame producers.  TEST INFRASTRUCTURE ONLY: the product never imports it.

``normalize_frames`` is the expression the reference's own test holds its kernel to
(tests/test_fused_operators.py:518-520: ``frames.astype(float32) / float32(255) * float32(2) - float32(1)``,
permuted to [cameras, 3, H, W]); it is therefore pinned by that test's formula.  ``frames_to_patches`` composes it
with the tensor expression of the SigLIP patch embedding (embodiinfer/policies/pi05/inference/vision.py:593-600).
"""

from __future__ import annotations

import numpy as np

from . import quant_oracle as Q


def normalize_frames(frames: np.ndarray) -> np.ndarray:
    """uint8 [cameras, H, W, 3] -> float32 [cameras, 3, H, W]."""
    host = frames.astype(np.float32) / np.float32(255) * np.float32(2) - np.float32(1)
    return np.ascontiguousarray(np.transpose(host, (0, 3, 1, 2)))


def frames_to_patches(frames: np.ndarray, patch: int) -> np.ndarray:
    """uint8 [cameras, H, W, 3] -> bf16 bits [cameras * gh * gw, 3 * patch * patch]
    (``images.bfloat16().view(b, 3, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(b * gh * gw, 3*p*p)``)."""
    images = normalize_frames(frames)
    cameras, _, height, width = images.shape
    grid_h, grid_w = height // patch, width // patch
    tiles = Q.f32_to_bf16(images).reshape(cameras, 3, grid_h, patch, grid_w, patch)
    return np.ascontiguousarray(np.transpose(tiles, (0, 2, 4, 1, 3, 5))).reshape(cameras * grid_h * grid_w, 3 * patch * patch)


def resample_axis(pixels: np.ndarray, bounds, weights, taps: int, axis: int) -> np.ndarray:
    """One pass of Pillow's 8-bit resample along ``axis`` (camera_frames.cu:32-54): 22-bit fixed-point taps, a
    half-unit rounding offset, arithmetic shift, clamp to a byte."""
    pixels = np.moveaxis(np.asarray(pixels, dtype=np.int64), axis, 0)
    outputs = len(bounds) // 2
    result = np.empty((outputs, *pixels.shape[1:]), dtype=np.uint8)
    for index in range(outputs):
        first, count = bounds[2 * index], bounds[2 * index + 1]
        tap = np.asarray(weights[index * taps: index * taps + count], dtype=np.int64)
        total = (1 << 21) + np.tensordot(tap, pixels[first:first + count], axes=(0, 0))
        result[index] = np.clip(total >> 22, 0, 255)
    return np.moveaxis(result, 0, axis)


def resize_with_pad(frames: np.ndarray, target: tuple[int, int], geometry, row_taps, column_taps) -> np.ndarray:
    """uint8 [cameras, H, W, 3] -> float32 [cameras, 3, *target]: horizontal pass, vertical pass, centred on a
    black canvas, normalised (camera_frames.cu:32-88).  ``geometry`` = (height, width, top, left);
    ``row_taps`` / ``column_taps`` = (bounds, weights, taps) of the horizontal / vertical axis."""
    height, width, top, left = geometry
    across = resample_axis(frames, *row_taps, axis=2)
    resized = resample_axis(across, *column_taps, axis=1)
    canvas = np.zeros((frames.shape[0], target[0], target[1], 3), dtype=np.uint8)
    canvas[:, top:top + height, left:left + width] = resized
    return normalize_frames(canvas)
