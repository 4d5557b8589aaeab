"""Device-side camera frame preparation: raw uint8 frames to normalised model images.

Drop-in for the reference's ``embodiinfer/backend/cuda/camera_frames.py`` (``normalize_frames``, ``FrameResize``:
same signatures, checks and error messages), on this package's kernels.  ``FrameResize`` reproduces OpenPI's
``resize_with_pad`` (Pillow's 8-bit two-pass bilinear resample onto a centred black canvas) bit for bit; the
fixed-point taps are computed on the host once per geometry with Pillow's published algorithm
(``precompute_coeffs`` / ``normalize_coeffs_8bpc`` of its Resample.c: a triangle filter widened by the downscale
factor, weights normalised in double precision, rounded half away from zero to 22 fractional bits).
"""

from __future__ import annotations

import math

import torch

from . import _native as N
from . import kernels as K
from .kernels import normalize_frames  # noqa: F401  (re-exported: the reference exposes it from this module)

PRECISION_BITS = 22


def pillow_bilinear_taps(source: int, target: int) -> tuple[list[int], list[int], int]:
    """Taps of one axis: ``bounds`` = [first source index, tap count] per output index (flattened), ``weights`` =
    ``taps`` fixed-point weights per output index (zero-padded), and ``taps``."""
    scale = source / target
    stretch = scale if scale > 1.0 else 1.0          # the filter is widened only when shrinking
    support = 1.0 * stretch                          # bilinear: a triangle of half-width 1
    taps = int(math.ceil(support)) * 2 + 1
    one = 1 << PRECISION_BITS
    bounds: list[int] = []
    weights: list[int] = []
    for position in range(target):
        centre = (position + 0.5) * scale
        first = int(centre - support + 0.5)
        first = first if first > 0 else 0
        last = int(centre + support + 0.5)
        last = last if last < source else source
        count = last - first
        triangle = []
        for offset in range(count):
            distance = (offset + first - centre + 0.5) * (1.0 / stretch)
            triangle.append(1.0 - abs(distance) if abs(distance) < 1.0 else 0.0)
        total = sum(triangle)
        if total != 0.0:
            triangle = [value / total for value in triangle]
        fixed = [int(value * one - 0.5) if value < 0 else int(value * one + 0.5) for value in triangle]
        bounds.extend((first, count))
        weights.extend(fixed + [0] * (taps - count))
    return bounds, weights, taps


def resize_geometry(source: tuple[int, int], target: tuple[int, int]) -> tuple[int, int, int, int]:
    """(resized height, resized width, top, left) of ``resize_with_pad``: one ratio fits the frame into the
    target, the result is centred."""
    ratio = max(source[1] / target[1], source[0] / target[0])
    height, width = int(source[0] / ratio), int(source[1] / ratio)
    return height, width, (target[0] - height) // 2, (target[1] - width) // 2


class FrameResize:
    """``resize_with_pad`` + ``(x / 255) * 2 - 1`` for frames of one (height, width), graph-capturable (the tap
    tables are uploaded once, here)."""

    def __init__(self, source: tuple[int, int], target: tuple[int, int], device: torch.device) -> None:
        self.source, self.canvas = tuple(source), tuple(target)
        self.height, self.width, self.top, self.left = resize_geometry(self.source, self.canvas)
        row_bounds, row_weights, self.row_taps = pillow_bilinear_taps(self.source[1], self.width)
        column_bounds, column_weights, self.column_taps = pillow_bilinear_taps(self.source[0], self.height)
        self.row_bounds, self.row_weights, self.column_bounds, self.column_weights = (
            torch.tensor(table, dtype=torch.int32, device=device)
            for table in (row_bounds, row_weights, column_bounds, column_weights)
        )

    def rows_buffer(self, cameras: int, device: torch.device) -> torch.Tensor:
        """The reference's scratch for its horizontal pass, [cameras, source height, resized width, 3] uint8.
        The kernel here needs none; the buffer exists so callers written for the reference keep working."""
        return torch.empty((cameras, self.source[0], self.width, 3), dtype=torch.uint8, device=device)

    def __call__(self, frames: torch.Tensor, rows: torch.Tensor | None, images: torch.Tensor) -> None:
        """Resize ``frames`` into ``images`` [cameras, 3, *target] on the current stream (``rows`` is unused)."""
        if frames.dtype != torch.uint8 or frames.ndim != 4 or frames.shape[3] != 3 or not frames.is_contiguous():
            raise ValueError("frames must be contiguous uint8 [cameras, height, width, 3]")
        if images.dtype != torch.float32 or images.ndim != 4 or tuple(images.shape[:2]) != (frames.shape[0], 3) or \
                not images.is_contiguous():
            raise ValueError("images must be contiguous float32 [cameras, 3, height, width]")
        if frames.device.type != "cuda" or images.device != frames.device:
            raise ValueError("frames and images must share a CUDA device")
        cameras = frames.shape[0]
        if tuple(frames.shape[1:3]) != self.source or tuple(images.shape[2:]) != self.canvas:
            raise ValueError("frames and images must match the planned source and target sizes")
        if rows is not None and (rows.dtype != torch.uint8 or tuple(rows.shape) != (cameras, self.source[0], self.width, 3)):
            raise ValueError("rows must be the uint8 scratch from rows_buffer")
        with torch.cuda.device(frames.device):
            status = N.load().b2_resize_frames(
                frames.data_ptr(), images.data_ptr(), self.row_bounds.data_ptr(), self.row_weights.data_ptr(), self.row_taps,
                self.column_bounds.data_ptr(), self.column_weights.data_ptr(), self.column_taps, cameras, self.source[0],
                self.source[1], self.height, self.width, self.canvas[0], self.canvas[1], self.top, self.left,
                K._stream(frames.device))
        if status:
            raise RuntimeError(f"Camera frame resize launch failed: {status}")
