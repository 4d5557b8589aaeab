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
