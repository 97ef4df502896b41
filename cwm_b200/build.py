"""Build the C-ABI shared library (``libcwm_b200.so``) for sm_100a with nvcc.

The library is built in-tree, next to this file, so that it travels with the
source tree.  ``python -m cwm_b200.build`` rebuilds it; ``build()`` only
rebuilds when a source is newer than the library.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libcwm_b200.so"
OBJ_DIR = PKG_DIR / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libcwm_b200.so")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _deps() -> list[Path]:
    return sources() + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "cwm_b200.h"]


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    lib_mtime = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > lib_mtime for p in _deps())


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(f"--- {src.name}\n{res.stdout}{res.stderr}", file=sys.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link ``libcwm_b200.so``; returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    OBJ_DIR.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose or ptxas_info, extra), sources()))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [
        _nvcc(), "-shared", "-o", str(tmp), *map(str, objs),
        "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
        "-Xcompiler", "-fPIC",
    ]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force=True, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(path)
