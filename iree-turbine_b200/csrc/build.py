"""Builds ``libb200kern.so`` (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Run as a script (``python build.py``) or call :func:`build`.  Objects are rebuilt only when a
source or header is newer than the object.  The library links the CUDA runtime statically and
does not link libcuda (the one driver entry it needs is resolved at run time), so it loads on a
machine without a GPU driver.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
REPO = PKG.parent
LIB_NAME = "libb200kern.so"
LIB_PATH = PKG / LIB_NAME
BUILD_DIR = CSRC / "build"

SOURCES = ["abi.cu", "gemm_sm100.cu", "gemm_splitk_sm100.cu", "attention_sm100.cu", "attention_tile_sm100.cu", "attention_bwd_sm100.cu", "decode_sm100.cu", "quant.cu", "selftest.cu"]
HEADERS = ["common.cuh", "ptx.cuh", "gemm_common.cuh", str(REPO / "include" / "b200k.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the CUDA kernel library")
    return cand


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: str, verbose: bool) -> Path:
    obj = BUILD_DIR / (Path(src).stem + ".o")
    deps = [CSRC / src] + [Path(h) if os.path.isabs(h) else CSRC / h for h in HEADERS]
    if _stale(obj, deps):
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        log = BUILD_DIR / (Path(src).stem + ".ptxas.log")
        log.write_text(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[build] compiled {src}")
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compiles every kernel translation unit and links the shared library.  Returns its path."""
    BUILD_DIR.mkdir(exist_ok=True)
    if force:
        for f in BUILD_DIR.glob("*.o"):
            f.unlink()
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    if force or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-Xcompiler", "-fPIC"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(f"[build] linked {LIB_PATH}")
    return LIB_PATH


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv)
    print(LIB_PATH)
