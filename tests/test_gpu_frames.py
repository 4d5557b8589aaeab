"""Camera-frame kernels against the CPU oracle (the reference test's own expression), bit-exact."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from embodiinfer_b200 import kernels as K
from oracle import frames_oracle as FO
from tests.util import bits

pytestmark = pytest.mark.gpu


def make_frames(cameras, height, width, seed):
    generator = torch.Generator().manual_seed(seed)
    frames = torch.randint(0, 256, (cameras, height, width, 3), dtype=torch.uint8, generator=generator)
    count = min(256, frames.numel())
    frames.view(-1)[:count] = torch.arange(count, dtype=torch.uint8)      # every byte value occurs in the larger cases
    return frames


@pytest.mark.parametrize("cameras,height,width", [(3, 224, 224), (1, 7, 5), (2, 480, 640)])
def test_normalize_frames(device, cameras, height, width):
    frames = make_frames(cameras, height, width, 41)
    images = torch.zeros((cameras, 3, height, width), device=device)
    K.normalize_frames(frames.to(device), images)
    assert np.array_equal(images.cpu().numpy().view(np.uint32), FO.normalize_frames(frames.numpy()).view(np.uint32))
    with pytest.raises(ValueError):
        K.normalize_frames(frames.to(device).float(), images)


@pytest.mark.parametrize("cameras,height,width,patch", [(3, 224, 224, 14), (2, 32, 48, 16), (1, 4, 6, 2)])
def test_frames_to_patches(device, cameras, height, width, patch):
    frames = make_frames(cameras, height, width, 43)
    rows = cameras * (height // patch) * (width // patch)
    patches = torch.zeros((rows, 3 * patch * patch), device=device, dtype=torch.bfloat16)
    K.frames_to_patches(frames.to(device), patches, patch)
    assert np.array_equal(bits(patches), FO.frames_to_patches(frames.numpy(), patch))
    # the same rows as the tensor expression of the patch embedding evaluated by torch on the device
    images = torch.zeros((cameras, 3, height, width), device=device)
    K.normalize_frames(frames.to(device), images)
    expected = images.bfloat16().view(cameras, 3, height // patch, patch, width // patch, patch).permute(0, 2, 4, 1, 3, 5)
    assert torch.equal(patches, expected.reshape(rows, 3 * patch * patch))


def test_frames_reject_bad_arguments(device):
    frames = torch.zeros((1, 15, 14, 3), device=device, dtype=torch.uint8)
    with pytest.raises((RuntimeError, ValueError)):      # height not a multiple of the patch
        K.frames_to_patches(frames, torch.zeros((1, 588), device=device, dtype=torch.bfloat16), 14)
    odd = torch.zeros((1, 3, 3, 3), device=device, dtype=torch.uint8)
    with pytest.raises(RuntimeError):                    # 3 * patch^2 must be a multiple of 4
        K.frames_to_patches(odd, torch.zeros((1, 27), device=device, dtype=torch.bfloat16), 3)


@pytest.mark.parametrize("source", [(256, 256), (480, 640), (128, 96), (224, 300), (224, 224)])
def test_frame_resize_matches_the_oracle(device, source):
    """Same sources as the reference's own test (tests/test_fused_operators.py:525); the oracle is pinned on Pillow."""
    from embodiinfer_b200.frames import FrameResize, pillow_bilinear_taps, resize_geometry
    frames = torch.randint(0, 256, (2, *source, 3), dtype=torch.uint8, generator=torch.Generator().manual_seed(0))
    resize = FrameResize(source, (224, 224), device)
    images = torch.empty((2, 3, 224, 224), device=device)
    resize(frames.to(device), resize.rows_buffer(2, device), images)
    geometry = resize_geometry(source, (224, 224))
    assert geometry == (resize.height, resize.width, resize.top, resize.left)
    want = FO.resize_with_pad(frames.numpy(), (224, 224), geometry, pillow_bilinear_taps(source[1], geometry[1]),
                              pillow_bilinear_taps(source[0], geometry[0]))
    assert np.array_equal(images.cpu().numpy().view(np.uint32), want.view(np.uint32))
    resize(frames.to(device), None, images)          # the scratch of the reference's two-pass kernel is optional here
    assert np.array_equal(images.cpu().numpy().view(np.uint32), want.view(np.uint32))
    with pytest.raises(ValueError):
        resize(frames.to(device)[:, :-1].contiguous(), None, images)
