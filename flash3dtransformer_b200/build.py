"""In-tree build of libf3d_b200.so with nvcc for sm_100a.

Every .cu file under csrc/ is compiled to an object (only when its sources changed) and linked into
flash3dtransformer_b200/lib/libf3d_b200.so.  No torch, pybind or glog dependency enters the library; it
links the static CUDA runtime only; driver entry points (cuTensorMapEncodeTiled) are resolved at run time
through cudaGetDriverEntryPoint, so the library also loads on a machine without a GPU driver.

Usage: python -m flash3dtransformer_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "lib"
OBJ_DIR = PKG / "csrc" / "build"
LIB = OUT_DIR / "libf3d_b200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return cand


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    deps = [src] + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    for d in deps:
        h.update(d.name.encode())
        h.update(d.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, force: bool, verbose: bool) -> tuple[Path, bool, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    dg = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == dg:
        return obj, False, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(dg)
    (OBJ_DIR / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    return obj, True, res.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError("no CUDA sources found")
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        results = list(ex.map(lambda s: _compile_one(s, force, verbose), sources))
    rebuilt = any(r[1] for r in results)
    for _, _, log in results:
        if log:
            print(log)
    if rebuilt or not LIB.exists():
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB),
               *[str(r[0]) for r in results]]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
