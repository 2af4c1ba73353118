"""Builds the parts of the REFERENCE that compile on a host, from the reference checkout where it lies, into
oracle/_ref/ (kept out of version control), and writes golden vectors from them.  TEST INFRASTRUCTURE ONLY: the
outputs pin oracle/psh_oracle.py and the library's scoreboard operator to the reference's own lines of code; nothing
in the product path loads them.

    python oracle/ref_build.py [<reference checkout>] [--golden]

  oracle/_ref/libf3d_ref_hash.so      the register overloads of vox_coord, h1_zorder_{div,mod}_3d, h1_xorsum_{div,mod}
                                      (src/psh/hash_fns.cuh:23-33,48-68,79-86,113-135, clamp from
                                      src/common/arithmetic.cuh:26-29), compiled by g++ through oracle/ref_hash_host.cpp
                                      with stand-ins for kittens.cuh / cub / rand.cuh (oracle/ref_stubs/)
  oracle/_ref/f3d_ref_sanitizer*.so   src/psh/bucket_sanitizer_cpu.cpp as a torch extension (glog stand-in from
                                      oracle/ref_stubs/), bound by oracle/ref_sanitizer_bind.cpp
  tests/golden/ref_hash.npz           (--golden) inputs and the reference's outputs for a fixed set of points and voxel
                                      triples, so that the pin also holds where no reference checkout exists

No reference source is copied: the compiler reads the files under <reference checkout>/src.  The rest of the
reference (kernels, dispatchers) needs ThunderKittens, glog and TransformerEngine and does not build here.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
STUBS = os.path.join(HERE, "ref_stubs")
HASH_LIB = os.path.join(OUT, "libf3d_ref_hash.so")
DEFAULT_REF = os.environ.get("F3D_REFERENCE", "/root/reference")


def have_reference(ref: str = DEFAULT_REF) -> bool:
    return os.path.isfile(os.path.join(ref, "src", "psh", "hash_fns.cuh"))


def build_hash(ref: str = DEFAULT_REF) -> str:
    os.makedirs(OUT, exist_ok=True)
    cmd = [shutil.which("g++") or "g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-w",
           "-I", STUBS, "-I", os.path.join(ref, "src"), os.path.join(HERE, "ref_hash_host.cpp"), "-o", HASH_LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"g++ failed on the reference's hash header:\n{res.stderr}")
    return HASH_LIB


def build_sanitizer(ref: str = DEFAULT_REF):
    """Compile the reference's bucket_sanitizer_cpu.cpp with torch's headers; returns the imported module."""
    from torch.utils import cpp_extension
    os.makedirs(OUT, exist_ok=True)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    return cpp_extension.load(
        name="f3d_ref_sanitizer",
        sources=[os.path.join(ref, "src", "psh", "bucket_sanitizer_cpu.cpp"), os.path.join(HERE, "ref_sanitizer_bind.cpp")],
        extra_include_paths=[STUBS, os.path.join(ref, "src"), cuda_inc],
        extra_cflags=["-O1", "-w"], build_directory=OUT, with_cuda=False, verbose=False)


def load_sanitizer():
    """Import an already built oracle/_ref/f3d_ref_sanitizer*.so (None when it has not been built)."""
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    for f in sorted(os.listdir(OUT)) if os.path.isdir(OUT) else []:
        if f.startswith("f3d_ref_sanitizer") and f.endswith(".so"):
            spec = importlib.util.spec_from_file_location("f3d_ref_sanitizer", os.path.join(OUT, f))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
    return None


class RefHash:
    """ctypes view of libf3d_ref_hash.so."""

    def __init__(self, path: str = HASH_LIB):
        self.lib = ctypes.CDLL(path)

    @staticmethod
    def _p(a):
        return a.ctypes.data_as(ctypes.c_void_p)

    def vox_hash(self, coord_f16, bbox_min_f16, bbox_max_f16, num_vox, divisor, num_bucket):
        """(vox u16 [n,3], hashes u16 [4,n]) of fp16 coordinates, by the reference's vox_coord + the four hashes."""
        c = np.ascontiguousarray(coord_f16, dtype=np.float16).astype(np.float32)
        lo = np.asarray(bbox_min_f16, dtype=np.float16).astype(np.float32)
        hi = np.asarray(bbox_max_f16, dtype=np.float16).astype(np.float32)
        n = c.shape[0]
        vox = np.zeros((n, 3), np.uint16)
        h = np.zeros((4, n), np.uint16)
        self.lib.f3d_ref_vox_hash(self._p(c), self._p(lo), self._p(hi), ctypes.c_uint32(num_vox), ctypes.c_uint64(n),
                                  ctypes.c_uint16(divisor), ctypes.c_uint16(num_bucket), self._p(vox), self._p(h))
        return vox, h

    def hash_of_vox(self, vox_u16, divisor, num_bucket):
        v = np.ascontiguousarray(vox_u16, dtype=np.uint16)
        n = v.shape[0]
        h = np.zeros((4, n), np.uint16)
        self.lib.f3d_ref_hash_of_vox(self._p(v), ctypes.c_uint64(n), ctypes.c_uint16(divisor), ctypes.c_uint16(num_bucket),
                                     self._p(h))
        return h


def golden_inputs():
    """Fixed inputs of tests/golden/ref_hash.npz: seeded points in a box (with the box corners and values next to voxel
    boundaries), a flat axis, and voxel triples covering every bit position and the extremes."""
    rng = np.random.default_rng(20240515)
    pts = (rng.random((1024, 3), dtype=np.float32) * np.float32([100, 100, 8]) - np.float32([50, 50, 2])).astype(np.float16)
    lo, hi = pts.min(0), pts.max(0)
    corners = np.array([[lo[0], lo[1], lo[2]], [hi[0], hi[1], hi[2]], [lo[0], hi[1], lo[2]], [hi[0], lo[1], hi[2]]], np.float16)
    mid = ((lo.astype(np.float32) + hi.astype(np.float32)) / 2).astype(np.float16)
    near = np.stack([np.nextafter(mid, np.float16(np.inf)), mid, np.nextafter(mid, np.float16(-np.inf))]).astype(np.float16)
    pts = np.concatenate([pts, corners, near])
    flat = pts[:64].copy()
    flat[:, 2] = np.float16(-1.5)
    bits = [0, 1, 0xFFFE, 0xFFFF, 0x8000, 0x7FFF, 0x0400, 0x0800, 0x03FF, 0x07FF, 0xAAAA, 0x5555]
    vox = np.array([(a, b, c) for a in bits for b in bits for c in bits], np.uint16)
    vox = np.concatenate([vox, rng.integers(0, 65536, (1024, 3)).astype(np.uint16)])
    return pts, flat, vox


def write_golden(ref: str = DEFAULT_REF) -> str:
    rh = RefHash(build_hash(ref))
    pts, flat, vox = golden_inputs()
    out = {"pts": pts, "flat": flat, "vox": vox}
    for nb in (128, 512, 2048):
        div = -(-0xFFFF // nb)
        v, h = rh.vox_hash(pts, pts.min(0), pts.max(0), 0xFFFF, div, nb)
        out["pts_vox"] = v
        out[f"pts_hash_{nb}"] = h
        vf, hf = rh.vox_hash(flat, flat.min(0), flat.max(0), 0xFFFF, div, nb)
        out["flat_vox"] = vf
        out[f"flat_hash_{nb}"] = hf
        out[f"vox_hash_{nb}"] = rh.hash_of_vox(vox, div, nb)
    path = os.path.join(os.path.dirname(HERE), "tests", "golden", "ref_hash.npz")
    np.savez_compressed(path, **out)
    return path


def build_all(ref: str = DEFAULT_REF, sanitizer: bool = True) -> None:
    build_hash(ref)
    if sanitizer:
        build_sanitizer(ref)


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    ref_dir = args[0] if args else DEFAULT_REF
    if not have_reference(ref_dir):
        raise SystemExit(f"{ref_dir} is not a reference checkout")
    build_all(ref_dir)
    print("built", sorted(os.listdir(OUT)))
    if "--golden" in sys.argv:
        print("wrote", write_golden(ref_dir))
