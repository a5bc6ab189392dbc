"""Build the native library in-tree: ``python -m megabake_b200.build``.

Compiles every ``csrc/*.cu`` for sm_100a with nvcc and links
``megabake_b200/_lib/libmegabake_b200.so`` (C ABI in ``include/megabake_b200.h``).
Cross-compiles without a GPU.  The build is skipped when the library is newer than
all of its sources unless ``force`` is given.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
LIB_DIR = PACKAGE / "_lib"
LIB_PATH = LIB_DIR / "libmegabake_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--fmad=false",  # keep fp32 multiply and add as the separate roundings the graph has
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build megabake_b200")
    return found


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps += list(INCLUDE.glob("*.h"))
    return any(path.stat().st_mtime > built for path in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objects = []
    for source in sources():
        obj = LIB_DIR / (source.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(source), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
        objects.append(str(obj))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objects, "-gencode",
           "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
