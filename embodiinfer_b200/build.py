"""Compile ``csrc/*.cu`` into ``libembodiinfer_b200.so`` next to this file (sm_100a only).

The library is built in-tree with ``nvcc`` and loaded with ``ctypes``; the same convention the
reference uses for its own kernels (embodiinfer/backend/cuda/native.py:43-119), minus the JIT
cache: the shared object travels with the package.
"""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
SOURCE_DIR = PACKAGE_DIR / "csrc"
LIBRARY_PATH = PACKAGE_DIR / "libembodiinfer_b200.so"
SOURCES = ("api.cu", "quantize.cu", "geglu.cu", "gemm.cu", "gemm_pair.cu", "gemm_skinny.cu", "static_scratch.cu", "rope.cu", "norm.cu", "frames.cu", "attention.cu")
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    if candidate.exists():
        return str(candidate)
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def sources() -> list[Path]:
    return [SOURCE_DIR / name for name in SOURCES if (SOURCE_DIR / name).exists()]


def is_stale() -> bool:
    if not LIBRARY_PATH.exists():
        return True
    built = LIBRARY_PATH.stat().st_mtime
    inputs = list(SOURCE_DIR.glob("*.cu")) + list(SOURCE_DIR.glob("*.cuh"))
    inputs.append(PACKAGE_DIR.parent / "include" / "embodiinfer_b200.h")
    return any(path.stat().st_mtime > built for path in inputs if path.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Build the shared library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIBRARY_PATH
    command = [
        nvcc_path(),
        *ARCH_FLAGS,
        "-lineinfo",
        "-O3",
        "-std=c++17",
        "--shared",
        "-Xcompiler",
        "-fPIC",
        "-o",
        str(LIBRARY_PATH),
        *[str(path) for path in sources()],
    ]
    command[1:1] = os.environ.get("B2_NVCC_FLAGS", "").split()      # e.g. -DB2_GEGLU_EPILOGUE_WARPS=8 to sweep the gated epilogue
    if verbose:
        command.insert(1, "-Xptxas=-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed ({result.returncode}):\n{result.stdout}\n{result.stderr}")
    if verbose:
        print(result.stderr)
    return LIBRARY_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
