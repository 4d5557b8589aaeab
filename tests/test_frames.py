"""Host side of the frame resize: the tap tables against the reference's own function (golden vectors) and the
numpy oracle of the two-pass resample against Pillow itself (the reference test's checker)."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

from embodiinfer_b200.frames import pillow_bilinear_taps, resize_geometry
from oracle import frames_oracle as FO

SOURCES = [(256, 256), (480, 640), (128, 96), (224, 300), (224, 224), (720, 1280)]


def test_taps_match_the_reference_function():
    golden = np.load(Path(__file__).parent / "golden" / "frames_golden.npz")
    for source, target in ((640, 298), (480, 224), (96, 168), (300, 224), (224, 224), (7, 3), (3, 7)):
        bounds, weights, taps = pillow_bilinear_taps(source, target)
        assert taps == int(golden[f"taps_{source}_{target}"])
        assert np.array_equal(np.asarray(bounds), golden[f"bounds_{source}_{target}"])
        assert np.array_equal(np.asarray(weights), golden[f"weights_{source}_{target}"])


@pytest.mark.parametrize("source", SOURCES)
def test_oracle_resize_matches_pillow(source):
    image_module = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(source[0] + source[1])
    frames = rng.integers(0, 256, (2, *source, 3), dtype=np.uint8)
    target = (224, 224)
    geometry = resize_geometry(source, target)
    got = FO.resize_with_pad(frames, target, geometry, pillow_bilinear_taps(source[1], geometry[1]),
                             pillow_bilinear_taps(source[0], geometry[0]))

    def resize_with_pad(image, size=224):          # the checker of the reference's own test, on Pillow
        original = image_module.fromarray(image)
        width, height = original.size
        ratio = max(width / size, height / size)
        resized = original.resize((int(width / ratio), int(height / ratio)), image_module.Resampling.BILINEAR)
        padded = image_module.new(original.mode, (size, size), 0)
        padded.paste(resized, ((size - resized.width) // 2, (size - resized.height) // 2))
        return np.asarray(padded)

    want = FO.normalize_frames(np.stack([resize_with_pad(frame) for frame in frames]))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
