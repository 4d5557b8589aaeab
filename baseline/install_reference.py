"""Install the unmodified reference package under ``baseline/_ref`` (git-ignored).

    python baseline/install_reference.py <path-to-the-reference-checkout>

The GPU tests that compare this library's kernels with the reference's own CUDA kernels
(``tests/test_gpu_reference_kernels.py``) and ``kernel_bench --reference`` import the package from there;
without the folder they skip.  Nothing is copied into the tracked tree.  The reference's build back end wants
to write into its source directory, so the install runs from a temporary copy.
"""

from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent
TARGET = ROOT / "_ref"


def install(source: Path) -> Path:
    if not (source / "pyproject.toml").exists():
        raise SystemExit(f"{source} is not a checkout of the reference (no pyproject.toml)")
    if TARGET.exists():
        shutil.rmtree(TARGET)
    with tempfile.TemporaryDirectory() as scratch:
        copy = Path(scratch) / "reference"
        shutil.copytree(source, copy, ignore=shutil.ignore_patterns(".git", "assets", "docs", "benchmarks"))
        command = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                   "--target", str(TARGET), str(copy)]
        subprocess.run(command, check=True)
    return TARGET


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(install(Path(sys.argv[1])))
