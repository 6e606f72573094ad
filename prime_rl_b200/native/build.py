"""Builds the native libraries in-tree.

``libprb200_cuda.so``  every ``csrc/*.cu`` compiled for sm_100a (nvcc cross-compiles on a host
                       without a GPU) and linked against the (static) CUDA runtime only;
``libprb200_cpu.so``   the C++ CPU optimizer (``csrc/cpu/*.cpp``), std::thread parallel.

Both expose a plain C ABI and are loaded through ``ctypes`` (see ``native/__init__.py``), so
there is no dependency on torch headers and a full rebuild takes well under a minute.

Run ``python -m prime_rl_b200.native.build`` to (re)build; objects are rebuilt only when
their source, or a header, is newer.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
OBJ = HERE / "build"
CUDA_LIB = HERE / "libprb200_cuda.so"
CPU_LIB = HERE / "libprb200_cpu.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add /usr/local/cuda/bin to PATH")


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _compile_cu(src: Path, headers_mtime: float, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, headers_mtime):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build_cuda(verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers_mtime = _newest(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_cu(s, headers_mtime, verbose), sources))
    if CUDA_LIB.exists() and CUDA_LIB.stat().st_mtime > _newest(objs):
        return CUDA_LIB
    cmd = [_nvcc(), "-shared", "-o", str(CUDA_LIB), *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return CUDA_LIB


def build_cpu() -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted((CSRC / "cpu").glob("*.cpp"))
    if not sources:
        return CPU_LIB
    if CPU_LIB.exists() and CPU_LIB.stat().st_mtime > _newest(sources):
        return CPU_LIB
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-fvisibility=hidden", "-o", str(CPU_LIB),
           *map(str, sources)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    return CPU_LIB


def build_all(verbose: bool = False) -> None:
    build_cuda(verbose)
    build_cpu()


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print(CUDA_LIB, CPU_LIB)
