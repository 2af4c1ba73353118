"""ctypes loader of libf3d_b200.so and the prototypes of its C ABI (include/f3d_b200.h).

There is no CPU fallback: if the shared library is missing or a call fails, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libf3d_b200.so"

_u32, _vp, _int, _f32 = c_uint32, c_void_p, c_int, c_float

# name -> (restype, argtypes); mirrors include/f3d_b200.h declaration by declaration
PROTOTYPES = {
    "f3d_last_error": (c_char_p, []),
    "f3d_version": (_int, []),
    "f3d_init_device": (_int, [_int]),
    "f3d_set_sync": (_int, [_int]),
    "f3d_get_sync": (_int, []),
    "f3d_set_seed": (_int, [c_uint64]),
    "f3d_get_seed": (c_uint64, []),
    "f3d_set_scene_base": (_int, [_u32]),
    "f3d_get_scene_base": (_u32, []),
    "f3d_release_workspaces": (_int, []),
    "f3d_launch_count": (ctypes.c_ulonglong, []),
    "f3d_batch_psh_scatter_pad_hash": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32,
                                              _vp, _vp, _vp, _vp, _vp, _u32, _f32, _u32, _int, _vp]),
    "f3d_batch_psh_scatter_pad_hash_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, _u32,
                                                      _vp, _vp, _vp, _vp, _vp, _u32, _f32, _u32, _int, _vp]),
    "f3d_batch_bucket_sanitizer_cpu": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32]),
    "f3d_batch_subbuck_reduce": (_int, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                        _vp, _u32, _u32, _u32, _int, _u32, _u32, _int, _vp]),
    "f3d_batch_subbuck_reduce_backward": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _u32, _u32, _int, _vp]),
    "f3d_additive_unpool_fwd": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _int, _u32, _int, _vp]),
    "f3d_additive_unpool_bwd": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _int, _u32, _int, _vp]),
    "f3d_device_status": (_int, [_int]),
    "f3d_linear_bf16": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _vp]),
    "f3d_linear_dtype": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _int, _vp]),
    "f3d_buck_swin_fwd_dtype": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _u32, _int, _int, _vp]),
    "f3d_linear_fused": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _vp, _vp, _f32, _vp, _int, _vp]),
    "f3d_row_stats_bf16": (_int, [_vp, _vp, _u32, _u32, _int, _vp]),
    "f3d_gemm_sm_bf16": (_int, [_vp, _vp, _vp, _int, _int, _int, _int, _vp]),
    "f3d_buck_swin_fwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int, _u32, _int, _vp]),
    "f3d_layernorm_bf16": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _f32, _int, _int, _vp]),
    "f3d_coord_embed_bf16": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _int, _vp]),
    "f3d_layernorm_bwd_bf16": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _f32, _int, _vp]),
    "f3d_swiglu_bwd_bf16": (_int, [_vp, _vp, _vp, c_uint64, _u32, _int, _vp]),
    "f3d_colsum_bf16": (_int, [_vp, _vp, c_uint64, _u32, _int, _vp]),
    "f3d_gelu_bwd_bf16": (_int, [_vp, _vp, _vp, c_uint64, _int, _int, _vp]),
    "f3d_coord_embed_bwd": (_int, [_vp, _vp, _vp, _vp, _u32, _u32, _int, _vp]),
    "f3d_linear_wgrad_bf16": (_int, [_vp, _vp, _vp, _vp, _int, _int, _int, _int, _vp]),
    "f3d_linear_ksplit_bf16": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _vp]),
    "f3d_collate_points_f32": (_int, [_vp, _vp, _vp, c_uint64, _u32, _int, _vp]),
    "f3d_scatter_index": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _int, _vp]),
    "f3d_gather_rows": (_int, [_vp, _vp, _vp, c_uint64, _u32, _u32, _int, _vp]),
    "f3d_buck_swin_bwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _int, _int, _int,
                                 _u32, _int, _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the library once; raise loudly when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flash3dtransformer_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def is_loaded() -> bool:
    return _lib is not None


def last_error() -> str:
    msg = load().f3d_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, what: str) -> None:
    """Turn a negative status into the RuntimeError the reference's bindings raise (std::runtime_error in
    src/common/runtime.h:36-86 surfaces as RuntimeError through pybind11)."""
    if status != 0:
        raise RuntimeError(f"{what}: {last_error()} (status {status})")
