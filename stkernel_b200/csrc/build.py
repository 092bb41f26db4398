"""Build the CUDA library in-tree: ``python -m stkernel_b200.csrc.build``.

Every ``.cu`` file here is compiled for sm_100a only and linked into
``stkernel_b200/_lib/libstk_b200.so`` (plain ``extern "C"`` entry points, loaded
with ctypes; no torch headers, so a file compiles in seconds and the library has
no ABI tie to a torch build).  Objects are rebuilt only when their source or a
header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE.parent / "_lib"
OBJ_DIR = HERE.parent.parent / "build" / "obj"
LIB = OUT_DIR / "libstk_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def sources() -> list[Path]:
    return sorted(HERE.glob("*.cu"))


def _newest_header() -> float:
    hs = list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = max(src.stat().st_mtime, _newest_header())
    if obj.exists() and obj.stat().st_mtime >= stamp:
        return obj
    cmd = ["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    if (not LIB.exists()) or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB),
               *[str(o) for o in objs], "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
