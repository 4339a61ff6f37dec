"""In-tree build of the sm_100a kernel library.

The kernels are plain CUDA with an ``extern "C"`` ABI (no torch headers), compiled with
``nvcc`` for ``sm_100a`` only and linked into ``libkhaosz_b200_kernels.so`` next to this
file.  ``python -m khaosz_b200.ops.build`` rebuilds; ``ensure_built()`` rebuilds only when
a source is newer than the library.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD_DIR = HERE / "build"
LIB_NAME = "libkhaosz_b200_kernels.so"
LIB_PATH = HERE / LIB_NAME

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdrs = _headers()
    jobs = []
    for src in sources():
        obj = BUILD_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + hdrs):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        (BUILD_DIR / (src.stem + ".ptxas.log")).write_text(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[build] {src.name}\n{res.stderr}", file=sys.stderr)
        return obj

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    objs = [BUILD_DIR / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def ensure_built() -> Path:
    """Build if needed and possible; return the library path (which may not exist when
    there is no nvcc and no prebuilt library)."""
    try:
        if _stale(LIB_PATH, sources() + _headers()):
            build()
    except RuntimeError:
        if not LIB_PATH.exists():
            raise
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(path)
