"""Builds `fxfusion_b200/lib/libfxf_b200.so` in-tree with nvcc for sm_100a.

    python -m fxfusion_b200.build [--force] [--verbose]

One shared library holds the C++17 runtime and every CUDA kernel; it links the CUDA runtime
statically and nothing from PyTorch.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libfxf_b200.so"
OBJ_DIR = PKG / "build"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build fxfusion_b200")
    return path


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cpp")) + sorted((CSRC / "kernels").glob("*.cu"))


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sources() + sorted(CSRC.glob("*.hpp")) + sorted((CSRC / "kernels").glob("*.cuh")) + [PKG.parent / "include" / "fxf_b200.h", Path(__file__)]:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [nvcc(), *ARCH, *COMMON, "-x", "cu", "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr, flush=True)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    stamp_file = LIB_DIR / "build.stamp"
    stamp = _stamp()
    if not force and LIB.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources()))
    cmd = [nvcc(), *ARCH, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static", "-ldl", "-Xlinker", "--no-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp_file.write_text(stamp)
    return LIB


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(out)
