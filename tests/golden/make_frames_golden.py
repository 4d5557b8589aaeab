"""Generate tests/golden/frames_golden.npz: the tap tables of the REFERENCE's own ``_pillow_bilinear_taps``
(embodiinfer/backend/cuda/camera_frames.py:64-90) for a few (source, target) axis lengths.

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_frames_golden.py
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

sys.dont_write_bytecode = True

from embodiinfer.backend.cuda.camera_frames import _pillow_bilinear_taps  # noqa: E402

OUT = Path(__file__).resolve().parent / "frames_golden.npz"


def main() -> None:
    arrays = {}
    for source, target in ((640, 298), (480, 224), (96, 168), (300, 224), (224, 224), (7, 3), (3, 7)):
        bounds, weights, taps = _pillow_bilinear_taps(source, target)
        arrays[f"bounds_{source}_{target}"] = np.asarray(bounds, dtype=np.int64)
        arrays[f"weights_{source}_{target}"] = np.asarray(weights, dtype=np.int64)
        arrays[f"taps_{source}_{target}"] = np.int64(taps)
    np.savez_compressed(OUT, **arrays)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
