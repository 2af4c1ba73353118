"""Operator module with the surface of the reference's pybind11 extension `flash3dxfmr.lib.pshattn`
(src/f3d_frontend.cu:112-138): same function names, same positional arguments, outputs mutated in place, errors
raised as RuntimeError.  Each function unpacks torch tensors into device pointers and calls the C ABI of
libf3d_b200.so (include/f3d_b200.h) on the tensor's device and torch's current stream.

The two attention entry points the reference's Python layer calls but whose bindings are commented out in its
snapshot (src/f3d_frontend.cu:136-137; callers flash3dxfmr/layers/buck_swin.py:57,91) are provided here.
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi

HASH_ZORDER_DIV, HASH_XORSUM_DIV, HASH_ZORDER_MOD, HASH_XORSUM_MOD = 1, 2, 3, 4
RED_MEAN, RED_SUM, RED_MIN, RED_MAX = 0, 1, 2, 3

_FEAT_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


# ------------------------------------------------------------------------------------------------ helpers
def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _check_tensors(tensors, names) -> torch.device:
    """assert_contiguous + assert_same_device of src/common/runtime.h:36-70.  (The checks run on every operator call of
    a forward pass, so the passing case is kept to plain comparisons; the messages are built only on failure.)"""
    dev = None
    for t, n in zip(tensors, names):
        if not isinstance(t, torch.Tensor):
            raise RuntimeError(f"{n} must be a torch.Tensor")
        if not t.is_contiguous():
            raise RuntimeError(f"Tensor {n} is not contiguous")
        if not t.is_cuda:
            raise RuntimeError(f"Tensor {n} is not on a CUDA device (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"Tensor {n} is on {t.device}, expected {dev}")
    return dev


def _check_dtype(tensors, names, dtype) -> None:
    """assert_dtype of src/common/runtime.h:72-86."""
    for t, n in zip(tensors, names):
        if t.dtype != dtype:
            raise RuntimeError(f"Tensor {n} has dtype {t.dtype}, expected {dtype}")


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(dev: torch.device) -> ctypes.c_void_p:
    """cudaStream_t of torch's current stream on the device."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(dev.index if dev.index is not None else torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _dev_index(dev: torch.device) -> int:
    return dev.index if dev.index is not None else torch.cuda.current_device()


# ------------------------------------------------------------------------------- DeviceManagerSingleton
class DeviceManagerSingleton:
    """Mirror of f3d::DeviceManagerSingleton (src/common/device_manager.cuh:25-64, bindings
    src/f3d_frontend.cu:115-120).  The reference keeps per-device cuRAND states and kernel dispatch tables here;
    this build needs neither (stateless RNG, compile-time kernel selection), so only the device check, the
    sync_stream flag and the seed remain."""
    _inst = None

    @staticmethod
    def instance() -> "DeviceManagerSingleton":
        if DeviceManagerSingleton._inst is None:
            DeviceManagerSingleton._inst = DeviceManagerSingleton()
        return DeviceManagerSingleton._inst

    def __init__(self) -> None:
        self._initialised = set()

    def init_dev_info(self, dev_id: int) -> None:
        if dev_id in self._initialised:
            return
        _cabi.check(_cabi.load().f3d_init_device(int(dev_id)), "init_dev_info")
        self._initialised.add(dev_id)

    def init_dispatchers(self) -> None:
        _cabi.load()

    def set_sync_stream(self, flag: bool) -> bool:
        # switching the flag off on a process that has not loaded the library yet is a no-op (off is the initial state):
        # building a model on a host without the CUDA library (the CPU restatement does) must not need it
        if not flag and not _cabi.is_loaded():
            return False
        return bool(_cabi.load().f3d_set_sync(1 if flag else 0))

    def get_sync_stream(self) -> bool:
        if not _cabi.is_loaded():
            return False
        return bool(_cabi.load().f3d_get_sync())

    # additions of this build
    def set_seed(self, seed: int) -> None:
        _cabi.check(_cabi.load().f3d_set_seed(int(seed) & 0xFFFFFFFFFFFFFFFF), "set_seed")

    def get_seed(self) -> int:
        return int(_cabi.load().f3d_get_seed())

    def set_scene_base(self, base: int) -> None:
        """Global index of this process's first scene (scene-sharded runs); enters the PSH random-number counter."""
        _cabi.check(_cabi.load().f3d_set_scene_base(int(base)), "set_scene_base")

    def get_scene_base(self) -> int:
        return int(_cabi.load().f3d_get_scene_base())


# ----------------------------------------------------------------------------------------------- PSH scatter
def batch_psh_scatter_pad_hash(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N,
                               num_bucket, bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max,
                               probe_offsets, cumsum_counter, scatter_coord, pad_num, hash_type) -> None:
    """f3d::batch_psh_scatter_pad_hash (src/psh/batch_psh_bucket_dispatcher.cu:221-326)."""
    names = ["coord", "bucket_id", "bucket_counter", "bucket_offset", "batch_sep", "probe_offsets",
             "cumsum_counter", "scatter_coord", "bbox_min", "bbox_max"]
    tensors = [coord, bucket_id, bucket_counter, bucket_offset, batch_sep, probe_offsets, cumsum_counter,
               scatter_coord, bbox_min, bbox_max]
    dev = _check_tensors(tensors, names)
    _check_dtype([coord, scatter_coord, bbox_min, bbox_max], ["coord", "scatter_coord", "bbox_min", "bbox_max"],
                 torch.float16)
    _check_dtype([bucket_counter, bucket_offset, batch_sep, cumsum_counter],
                 ["bucket_counter", "bucket_offset", "batch_sep", "cumsum_counter"], torch.uint32)
    _check_dtype([bucket_id], ["bucket_id"], torch.uint16)
    _check_dtype([probe_offsets], ["probe_offsets"], torch.int16)
    _require(coord.dim() == 2 and coord.shape[1] == 3, f"coord must be [N,3], got {tuple(coord.shape)}")
    _require(scatter_coord.dim() == 2 and scatter_coord.shape[1] == 3, "scatter_coord must be [pad_to,3]")
    total_n = coord.shape[0]
    batch = batch_sep.shape[0]
    _require(bucket_id.numel() >= total_n and bucket_offset.numel() >= total_n,
             "bucket_id / bucket_offset are shorter than coord")
    _require(bucket_counter.numel() == batch * num_bucket and cumsum_counter.numel() == batch * num_bucket,
             f"bucket_counter / cumsum_counter must be [{batch},{num_bucket}]")
    _require(probe_offsets.numel() == 128 * 3, "probe_offsets must be [128,3]")
    _require(bbox_min.numel() == 3 and bbox_max.numel() == 3, "bbox_min / bbox_max must have 3 elements")
    st = _cabi.load().f3d_batch_psh_scatter_pad_hash(
        _ptr(coord), _ptr(bucket_id), _ptr(bucket_counter), _ptr(bucket_offset), _ptr(batch_sep),
        total_n, batch, int(instance_max_N), int(num_bucket), int(bucket_divisor), int(bucket_size), int(num_vox),
        _ptr(bbox_min), _ptr(bbox_max), _ptr(probe_offsets), _ptr(cumsum_counter), _ptr(scatter_coord),
        scatter_coord.shape[0], float(pad_num), int(hash_type), _dev_index(dev), _stream(dev))
    _cabi.check(st, "batch_psh_scatter_pad_hash")


def batch_psh_scatter_pad(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N, num_bucket,
                          bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets, cumsum_counter,
                          scatter_coord, pad_num) -> None:
    """f3d::batch_psh_scatter_pad (src/psh/batch_psh_bucket_dispatcher.cu:123-219): Z-order-mod hash."""
    batch_psh_scatter_pad_hash(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N,
                               num_bucket, bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets,
                               cumsum_counter, scatter_coord, pad_num, HASH_ZORDER_MOD)


def batch_psh_scatter(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N, num_bucket,
                      bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets, cumsum_counter,
                      scatter_coord, hash_dtype=None, coord_dtype=None, block_size_N=1024) -> None:
    """f3d::batch_psh_scatter (src/psh/batch_psh_bucket_dispatcher.cu:39-121): Z-order-mod hash, no tail padding
    beyond what scatter_coord holds.  hash_dtype, coord_dtype and block_size_N are accepted and ignored, as the
    dtypes are fixed (u16 / fp16) and the tile size is chosen by the library."""
    batch_psh_scatter_pad_hash(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N,
                               num_bucket, bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max, probe_offsets,
                               cumsum_counter, scatter_coord, 0.0, HASH_ZORDER_MOD)


# --------------------------------------------------------------------------------------- scoreboard check
def batch_bucket_sanitizer_cpu(bucket_id, bucket_counter, bucket_offset, offset_check_table, bucket_residual,
                               batch_sep, offset_maxcnt, batch_size, num_bucket) -> None:
    """f3d::batch_bucket_sanitizer_cpu (src/psh/bucket_sanitizer_cpu.cpp:92-176; call site tests/test_psh.py:127-129).
    The scoreboard check of a finished bucketing, on the host: tensors of any device are copied to the CPU (as the
    reference does, :104-110), every point takes one unit off `bucket_residual[scene, bucket]` and marks
    `offset_check_table[scene, bucket, offset]`; every slot below a bucket's count must end up marked exactly once.
    `bucket_residual` and `offset_check_table` are updated in place on their own device (:172-173).  A violation
    raises RuntimeError naming the first offending point or slot."""
    tensors = [bucket_id, bucket_counter, bucket_offset, offset_check_table, bucket_residual, batch_sep, offset_maxcnt]
    names = ["bucket_id", "bucket_counter", "bucket_offset", "offset_check_table", "bucket_residual", "batch_sep",
             "offset_maxcnt"]
    for t, n in zip(tensors, names):
        _require(isinstance(t, torch.Tensor), f"{n} must be a torch.Tensor")
    _check_dtype([bucket_id], ["bucket_id"], torch.uint16)
    _check_dtype([bucket_counter, bucket_offset, bucket_residual, batch_sep, offset_maxcnt],
                 ["bucket_counter", "bucket_offset", "bucket_residual", "batch_sep", "offset_maxcnt"], torch.uint32)
    _check_dtype([offset_check_table], ["offset_check_table"], torch.int8)
    batch_size, num_bucket = int(batch_size), int(num_bucket)
    _require(offset_check_table.dim() == 3 and offset_check_table.shape[0] == batch_size
             and offset_check_table.shape[1] == num_bucket,
             f"offset_check_table must be [{batch_size},{num_bucket},max_count], got {tuple(offset_check_table.shape)}")
    _require(bucket_counter.numel() == batch_size * num_bucket and bucket_residual.numel() == batch_size * num_bucket,
             f"bucket_counter / bucket_residual must be [{batch_size},{num_bucket}]")
    _require(batch_sep.numel() >= batch_size and offset_maxcnt.numel() >= batch_size,
             "batch_sep / offset_maxcnt are shorter than batch_size")
    _require(bucket_offset.numel() >= bucket_id.numel(), "bucket_offset is shorter than bucket_id")
    host = [t.detach().cpu().contiguous() for t in tensors]
    # the two in/out buffers are private host copies even for CPU inputs, so a failed check changes nothing
    table, residual = host[3].clone(), host[4].clone()
    st = _cabi.load().f3d_batch_bucket_sanitizer_cpu(
        _ptr(host[0]), _ptr(host[1]), _ptr(host[2]), _ptr(table), _ptr(residual), _ptr(host[5]), _ptr(host[6]),
        bucket_id.numel(), batch_size, num_bucket, offset_check_table.shape[2])
    _cabi.check(st, "batch_bucket_sanitizer_cpu")
    bucket_residual.copy_(residual.view(bucket_residual.shape))
    offset_check_table.copy_(table)


# ------------------------------------------------------------------------------------- pooling / unpooling
def _feat_code(t: torch.Tensor, name: str) -> int:
    _require(t.dtype in _FEAT_DTYPES, f"Tensor {name} has dtype {t.dtype}; bfloat16, float16 and float32 are supported")
    return _FEAT_DTYPES[t.dtype]


def batch_subbuck_reduce(scattered_coord, scattered_feat, batch_sep, instance_max_N, subbuck_size, num_vox,
                         bbox_min, bbox_max, subbuck_id, subbuck_off, reduced_batch_sep, reduced_coord,
                         reduced_feat, unpool_ind, hash_type, red_op) -> None:
    """f3d::batch_subbuck_reduce (src/psh/batch_subbuck_pooling_dispatcher.cu:35-144)."""
    names = ["scattered_coord", "scattered_feat", "batch_sep", "subbuck_id", "subbuck_off", "reduced_batch_sep",
             "reduced_coord", "reduced_feat", "unpool_ind", "bbox_min", "bbox_max"]
    tensors = [scattered_coord, scattered_feat, batch_sep, subbuck_id, subbuck_off, reduced_batch_sep,
               reduced_coord, reduced_feat, unpool_ind, bbox_min, bbox_max]
    dev = _check_tensors(tensors, names)
    code = _feat_code(scattered_feat, "scattered_feat")
    _check_dtype([reduced_feat], ["reduced_feat"], scattered_feat.dtype)
    _check_dtype([scattered_coord, reduced_coord, bbox_min, bbox_max],
                 ["scattered_coord", "reduced_coord", "bbox_min", "bbox_max"], torch.float16)
    _check_dtype([batch_sep, subbuck_id, reduced_batch_sep, unpool_ind],
                 ["batch_sep", "subbuck_id", "reduced_batch_sep", "unpool_ind"], torch.uint32)
    _check_dtype([subbuck_off], ["subbuck_off"], torch.uint16)
    _require(scattered_feat.shape[1] == reduced_feat.shape[1],
             f"Input feature dim({scattered_feat.shape[1]}) != output feature dim({reduced_feat.shape[1]}).")
    _require(reduced_coord.shape[0] == reduced_feat.shape[0],
             f"Reduced coordinate length({reduced_coord.shape[0]}) != reduced feature length({reduced_feat.shape[0]}).")
    _require(scattered_coord.shape[1] == 3 and reduced_coord.shape[1] == 3,
             f"Input coordinates dim({scattered_coord.shape[1]}) or reduced coordinates dim({reduced_coord.shape[1]}) "
             "are NOT 3D.")
    _require(0 <= int(red_op) <= 3, f"Unsupported reduction operation id-{red_op}")
    _require(unpool_ind.dim() == 2 and unpool_ind.shape[1] == subbuck_size,
             f"Unpool_ind last dimension({unpool_ind.shape[-1]}) != subbucket_size({subbuck_size})")
    total_n = scattered_coord.shape[0]
    _require(scattered_feat.shape[0] >= total_n, "scattered_feat has fewer rows than scattered_coord")
    _require(subbuck_id.numel() >= total_n and subbuck_off.numel() >= total_n, "subbuck_id / subbuck_off too short")
    _require(reduced_batch_sep.shape[0] == batch_sep.shape[0], "reduced_batch_sep and batch_sep differ in length")
    st = _cabi.load().f3d_batch_subbuck_reduce(
        _ptr(scattered_coord), _ptr(scattered_feat), _ptr(batch_sep), total_n, batch_sep.shape[0],
        int(instance_max_N), int(subbuck_size), int(num_vox), _ptr(bbox_min), _ptr(bbox_max), _ptr(subbuck_id),
        _ptr(subbuck_off), _ptr(reduced_batch_sep), _ptr(reduced_coord), _ptr(reduced_feat), _ptr(unpool_ind),
        unpool_ind.shape[0], reduced_feat.shape[0], scattered_feat.shape[1], code, int(hash_type), int(red_op),
        _dev_index(dev), _stream(dev))
    _cabi.check(st, "batch_subbuck_reduce")


def batch_subbuck_reduce_backward(grad_red_feat, input_feat, unpool_ind, grad_input_feat, subbuck_size,
                                  reduction_op) -> None:
    """f3d::batch_subbuck_reduce_backward (src/psh/batch_subbuck_pooling_bwd_dispatcher.cu:26-85)."""
    dev = _check_tensors([grad_red_feat, input_feat, unpool_ind, grad_input_feat],
                         ["grad_red_feat", "input_feat", "unpool_ind", "grad_input_feat"])
    code = _feat_code(input_feat, "input_feat")
    _check_dtype([grad_red_feat, grad_input_feat], ["grad_red_feat", "grad_input_feat"], input_feat.dtype)
    _check_dtype([unpool_ind], ["unpool_ind"], torch.uint32)
    _require(unpool_ind.dim() == 2 and unpool_ind.shape[1] == subbuck_size,
             f"Unpool_ind last dimension({unpool_ind.shape[-1]}) != subbucket_size({subbuck_size})")
    _require(grad_red_feat.shape[0] >= unpool_ind.shape[0], "grad_red_feat has fewer rows than unpool_ind")
    _require(grad_red_feat.shape[1] == input_feat.shape[1] == grad_input_feat.shape[1], "feature dims differ")
    _require(grad_input_feat.shape[0] == input_feat.shape[0], "grad_input_feat and input_feat differ in length")
    _require(0 <= int(reduction_op) <= 3, f"Unsupported reduction_op={reduction_op}")
    st = _cabi.load().f3d_batch_subbuck_reduce_backward(
        _ptr(grad_red_feat), _ptr(input_feat), _ptr(unpool_ind), _ptr(grad_input_feat), input_feat.shape[0],
        unpool_ind.shape[0], input_feat.shape[1], code, int(subbuck_size), int(reduction_op), _dev_index(dev),
        _stream(dev))
    _cabi.check(st, "batch_subbuck_reduce_backward")


def additive_unpool_fwd(res_feat, down_feat, up_add_feat, unpool_ind, subbuck_size, covered_rows=None) -> None:
    """f3d::additive_unpool_fwd (src/psh/additive_unpool_dispatcher.cu:26-79).  `covered_rows` (not in the
    reference) is the number of leading rows that unpool_ind refers to; rows behind it are zero-filled instead of
    being left uninitialised.  None keeps the reference behaviour."""
    dev = _check_tensors([res_feat, down_feat, up_add_feat, unpool_ind],
                         ["res_feat", "down_feat", "up_add_feat", "unpool_ind"])
    code = _feat_code(res_feat, "res_feat")
    _check_dtype([down_feat, up_add_feat], ["down_feat", "up_add_feat"], res_feat.dtype)
    _check_dtype([unpool_ind], ["unpool_ind"], torch.uint32)
    _require(unpool_ind.dim() == 2 and unpool_ind.shape[1] == subbuck_size,
             f"Unpool_ind last dimension({unpool_ind.shape[-1]}) != subbucket_size({subbuck_size})")
    _require(res_feat.shape == up_add_feat.shape, "res_feat and up_add_feat differ in shape")
    _require(down_feat.shape[0] >= unpool_ind.shape[0], "down_feat has fewer rows than unpool_ind")
    _require(down_feat.shape[1] == res_feat.shape[1], "feature dims differ")
    up_rows = res_feat.shape[0]
    st = _cabi.load().f3d_additive_unpool_fwd(
        _ptr(res_feat), _ptr(down_feat), _ptr(up_add_feat), _ptr(unpool_ind), up_rows, unpool_ind.shape[0],
        up_rows if covered_rows is None else int(covered_rows), res_feat.shape[1], code, int(subbuck_size),
        _dev_index(dev), _stream(dev))
    _cabi.check(st, "additive_unpool_fwd")


def additive_unpool_bwd(grad_res, grad_down, grad_up_added, unpool_ind, subbuck_size) -> None:
    """f3d::additive_unpool_bwd (src/psh/additive_unpool_dispatcher.cu:81-134)."""
    dev = _check_tensors([grad_res, grad_down, grad_up_added, unpool_ind],
                         ["grad_res", "grad_down", "grad_up_added", "unpool_ind"])
    code = _feat_code(grad_up_added, "grad_up_added")
    _check_dtype([grad_res, grad_down], ["grad_res", "grad_down"], grad_up_added.dtype)
    _check_dtype([unpool_ind], ["unpool_ind"], torch.uint32)
    _require(unpool_ind.dim() == 2 and unpool_ind.shape[1] == subbuck_size,
             f"Unpool_ind last dimension({unpool_ind.shape[-1]}) != subbucket_size({subbuck_size})")
    _require(grad_res.shape == grad_up_added.shape, "grad_res and grad_up_added differ in shape")
    _require(grad_down.shape[0] >= unpool_ind.shape[0], "grad_down has fewer rows than unpool_ind")
    st = _cabi.load().f3d_additive_unpool_bwd(
        _ptr(grad_res), _ptr(grad_down), _ptr(grad_up_added), _ptr(unpool_ind), grad_up_added.shape[0],
        unpool_ind.shape[0], grad_up_added.shape[1], code, int(subbuck_size), _dev_index(dev), _stream(dev))
    _cabi.check(st, "additive_unpool_bwd")


# ------------------------------------------------------------------------------------------------- GEMMs
EPI_NONE, EPI_GELU, EPI_SWIGLU = 0, 1, 2


def device_status(device=None) -> None:
    """Raise if a kernel of this library abandoned a bounded wait on `device` since the last check."""
    idx = torch.cuda.current_device() if device is None else _dev_index(torch.device(device))
    _cabi.check(_cabi.load().f3d_device_status(idx), "device_status")


def gemm_sm_bf16(A, B, O) -> None:
    """f3d::gemm_sm_bf16 (src/psh/gemm_dispatcher.cu:26-80): O[M,N] = A[M,K] @ B[K,N], bf16."""
    dev = _check_tensors([A, B, O], ["A", "B", "O"])
    _check_dtype([A, B, O], ["A", "B", "O"], torch.bfloat16)
    _require(A.dim() == 2 and B.dim() == 2 and O.dim() == 2, "A, B, O must be matrices")
    m, k = A.shape
    _require(B.shape[0] == k, f"A is [{m},{k}] but B is {tuple(B.shape)}")
    n = B.shape[1]
    _require(tuple(O.shape) == (m, n), f"O must be [{m},{n}], got {tuple(O.shape)}")
    _cabi.check(_cabi.load().f3d_gemm_sm_bf16(_ptr(A), _ptr(B), _ptr(O), m, n, k, _dev_index(dev), _stream(dev)),
                "gemm_sm_bf16")


def linear_bf16(x, weight, bias, out, residual=None, nsplit=1, epilogue=EPI_NONE) -> None:
    """out = x @ weight^T (+ bias) (+ residual) on the tcgen05 GEMM; `out` holds nsplit contiguous
    [M, N/nsplit] matrices (nsplit=3: Q, K, V).  x, weight, residual and out share one element type, bfloat16 or
    float16 (float16 is the element type of the reference's CPU-runnable configuration; forward only).  Not part of
    the reference's operator module: the reference leaves these projections to nn.Linear / cuBLAS
    (flash3dxfmr/layers/buck_swin.py:159,163)."""
    tensors, names = [x, weight, out], ["x", "weight", "out"]
    if residual is not None:
        tensors.append(residual); names.append("residual")
    dev = _check_tensors(tensors, names)
    _require(x.dtype in (torch.bfloat16, torch.float16), f"Tensor x has dtype {x.dtype}; bfloat16 and float16 are supported")
    _check_dtype(tensors, names, x.dtype)
    m, k = x.shape
    n = weight.shape[0]
    _require(weight.shape[1] == k, f"weight must be [N,{k}], got {tuple(weight.shape)}")
    out_n = n // 2 if epilogue == EPI_SWIGLU else n
    _require(out.numel() == m * out_n, f"out must hold {m}x{out_n} elements, got {out.numel()}")
    bptr = ctypes.c_void_p(0)
    if bias is not None:
        _check_tensors([bias], ["bias"])
        _check_dtype([bias], ["bias"], torch.float32)
        _require(bias.numel() == n, f"bias must have {n} elements")
        bptr = _ptr(bias)
    rptr = ctypes.c_void_p(0)
    if residual is not None:
        _require(tuple(residual.shape) == (m, out_n), f"residual must be [{m},{out_n}]")
        rptr = _ptr(residual)
    st = _cabi.load().f3d_linear_dtype(_ptr(x), _ptr(weight), bptr, rptr, _ptr(out), m, n, k, int(nsplit), int(epilogue),
                                       _FEAT_DTYPES[x.dtype], _dev_index(dev), _stream(dev))
    _cabi.check(st, "linear_bf16")


linear = linear_bf16          # the element type follows the tensors


def linear_fused(x, weight, bias, out, residual=None, nsplit=1, epilogue=EPI_NONE, ln_stats=None, ln_colsum=None,
                 ln_eps=1e-5, stats_out=None) -> None:
    """linear_bf16 with a LayerNorm folded in (`ln_stats` fp32 [M, 2] row sums of x, `weight` already scaled by the
    LayerNorm weight, `ln_colsum` fp32 [N] its row sums, `bias` fp32 [N] with the LayerNorm bias folded in) and / or the
    row sums of the output written to `stats_out` fp32 [M, 2] for the LayerNorm that follows.  See f3d_linear_fused."""
    tensors, names = [x, weight, out], ["x", "weight", "out"]
    for t, n in ((residual, "residual"),):
        if t is not None:
            tensors.append(t); names.append(n)
    dev = _check_tensors(tensors, names)
    _require(x.dtype in (torch.bfloat16, torch.float16), f"Tensor x has dtype {x.dtype}; bfloat16 and float16 are supported")
    _check_dtype(tensors, names, x.dtype)
    m, k = x.shape
    n = weight.shape[0]
    _require(weight.shape[1] == k, f"weight must be [N,{k}], got {tuple(weight.shape)}")
    out_n = n // 2 if epilogue == EPI_SWIGLU else n
    _require(out.numel() == m * out_n, f"out must hold {m}x{out_n} elements, got {out.numel()}")
    _require(residual is None or tuple(residual.shape) == (m, out_n), f"residual must be [{m},{out_n}]")
    f32 = [t for t in (bias, ln_stats, ln_colsum, stats_out) if t is not None]
    if f32:
        _check_tensors(f32, ["fp32 side input"] * len(f32))
        _check_dtype(f32, ["fp32 side input"] * len(f32), torch.float32)
    _require(bias is None or bias.numel() == n, f"bias must have {n} elements")
    if ln_stats is not None:
        _require(ln_colsum is not None and bias is not None, "a folded LayerNorm needs ln_colsum and the folded bias")
        _require(ln_stats.numel() == 2 * m and ln_colsum.numel() == n, f"ln_stats must be [{m},2] and ln_colsum [{n}]")
    _require(stats_out is None or stats_out.numel() == 2 * m, f"stats_out must be [{m},2]")
    opt = lambda t: _ptr(t) if t is not None else ctypes.c_void_p(0)
    st = _cabi.load().f3d_linear_fused(_ptr(x), _ptr(weight), opt(bias), opt(residual), _ptr(out), m, n, k, int(nsplit),
                                       int(epilogue), _FEAT_DTYPES[x.dtype], opt(ln_stats), opt(ln_colsum), float(ln_eps),
                                       opt(stats_out), _dev_index(dev), _stream(dev))
    _cabi.check(st, "linear_fused")


def row_stats_bf16(x, stats) -> None:
    """stats fp32 [rows, 2] = (sum, sum of squares) of every row of x bf16 [rows, C]."""
    dev = _check_tensors([x, stats], ["x", "stats"])
    _check_dtype([x], ["x"], torch.bfloat16)
    _check_dtype([stats], ["stats"], torch.float32)
    _require(x.dim() == 2 and stats.numel() == 2 * x.shape[0], "x must be [rows, C] and stats [rows, 2]")
    st = _cabi.load().f3d_row_stats_bf16(_ptr(x), _ptr(stats), x.shape[0], x.shape[1], _dev_index(dev), _stream(dev))
    _cabi.check(st, "row_stats_bf16")


def wgrad_supported(n: int, k: int) -> bool:
    """Shapes linear_wgrad_bf16 takes: N a multiple of 8, K = 32 or a multiple of 64."""
    return n % 8 == 0 and (k == 32 or k % 64 == 0)


def linear_wgrad_bf16(grad_out, x, grad_weight, grad_bias=None) -> None:
    """grad_weight fp32 [N, K] = grad_out^T @ x and grad_bias fp32 [N] = grad_out.sum(0) for bf16 grad_out [M, N] and
    x [M, K]: the parameter gradients of a projection in one pass over both operands, added in a fixed order."""
    ts, names = [grad_out, x, grad_weight], ["grad_out", "x", "grad_weight"]
    if grad_bias is not None:
        ts.append(grad_bias); names.append("grad_bias")
    dev = _check_tensors(ts, names)
    _check_dtype([grad_out, x], ["grad_out", "x"], torch.bfloat16)
    _check_dtype(ts[2:], names[2:], torch.float32)
    _require(grad_out.dim() == 2 and x.dim() == 2 and grad_out.shape[0] == x.shape[0], "grad_out must be [M, N] and x [M, K]")
    m, n = grad_out.shape
    k = x.shape[1]
    _require(tuple(grad_weight.shape) == (n, k), f"grad_weight must be [{n},{k}]")
    _require(grad_bias is None or grad_bias.numel() == n, f"grad_bias must have {n} elements")
    st = _cabi.load().f3d_linear_wgrad_bf16(_ptr(grad_out), _ptr(x), _ptr(grad_weight), _ptr(grad_bias) if grad_bias is not None else None,
                                            m, n, k, _dev_index(dev), _stream(dev))
    _cabi.check(st, "linear_wgrad_bf16")


def linear_ksplit_bf16(x, weight, out, bias=None, residual=None) -> None:
    """out [M, N] = sum_s x[s] @ weight[s]^T for x bf16 [S, M, K] and weight bf16 [S, N, K]: the input gradient of a
    projection whose output is S separate matrices (Q, K, V), computed from the packed gradient in one GEMM."""
    tensors, names = [x, weight, out], ["x", "weight", "out"]
    if residual is not None:
        tensors.append(residual); names.append("residual")
    dev = _check_tensors(tensors, names)
    _check_dtype(tensors, names, torch.bfloat16)
    _require(x.dim() == 3 and weight.dim() == 3 and x.shape[0] == weight.shape[0] and x.shape[2] == weight.shape[2],
             f"x must be [S, M, K] and weight [S, N, K], got {tuple(x.shape)} and {tuple(weight.shape)}")
    s, m, k = x.shape
    n = weight.shape[1]
    _require(tuple(out.shape) == (m, n), f"out must be [{m},{n}]")
    _require(residual is None or tuple(residual.shape) == (m, n), f"residual must be [{m},{n}]")
    bptr = ctypes.c_void_p(0)
    if bias is not None:
        _check_tensors([bias], ["bias"])
        _check_dtype([bias], ["bias"], torch.float32)
        _require(bias.numel() == n, f"bias must have {n} elements")
        bptr = _ptr(bias)
    st = _cabi.load().f3d_linear_ksplit_bf16(_ptr(x), _ptr(weight), bptr, _ptr(residual) if residual is not None else None,
                                             _ptr(out), m, n, k, s, _dev_index(dev), _stream(dev))
    _cabi.check(st, "linear_ksplit_bf16")


# --------------------------------------------------------------------------------------- bucketed attention
def _check_qkv(tensors, names, dtypes=(torch.bfloat16,)):
    dev = _check_tensors(tensors, names)
    _require(tensors[0].dtype in dtypes, f"Tensor {names[0]} has dtype {tensors[0].dtype}; supported: {', '.join(str(d) for d in dtypes)}")
    _check_dtype(tensors, names, tensors[0].dtype)
    shape = tuple(tensors[0].shape)
    _require(len(shape) == 4, f"Expect {names[0]} with four axes [B, L, H, D], but got shape={shape}")
    for t, n in zip(tensors, names):
        _require(tuple(t.shape) == shape, f"{n} has shape {tuple(t.shape)}, expected {shape}")
    return dev, shape


def buck_swin_fwd(Q, K, V, O, L, Scope_buckets, bucket_size) -> None:
    """f3d::buck_swin_fwd (declared src/f3d_frontend.cu:90-92; caller flash3dxfmr/layers/buck_swin.py:57).
    O[B,L,H,D] and the log-sum-exp L[B,L,H] are written in place.  Q, K, V, O are bfloat16 or float16 (all the
    same)."""
    dev, (b, l, h, d) = _check_qkv([Q, K, V, O], ["Q", "K", "V", "O"], (torch.bfloat16, torch.float16))
    _check_tensors([L, Scope_buckets], ["L", "Scope_buckets"])
    _check_dtype([L], ["L"], torch.float32)
    _check_dtype([Scope_buckets], ["Scope_buckets"], torch.uint32)
    _require(tuple(L.shape) == (b, l, h), f"L must be [{b},{l},{h}], got {tuple(L.shape)}")
    _require(Scope_buckets.dim() == 2, "Scope_buckets must be [num_scopes, scope_size]")
    st = _cabi.load().f3d_buck_swin_fwd_dtype(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(L), _ptr(Scope_buckets), b, l, h, d,
                                              Scope_buckets.shape[0], Scope_buckets.shape[1], int(bucket_size),
                                              _FEAT_DTYPES[Q.dtype], _dev_index(dev), _stream(dev))
    _cabi.check(st, "buck_swin_fwd")


def layernorm_bf16(x, weight, bias, out, eps=1e-5, gelu=False) -> None:
    """out = LayerNorm(x) (optionally followed by GELU) over the last dimension; x/out bf16 [rows, C], weight/bias
    fp32 [C].  Not part of the reference's operator module (it uses te.LayerNorm / nn.LayerNorm)."""
    dev = _check_tensors([x, weight, bias, out], ["x", "weight", "bias", "out"])
    _check_dtype([x, out], ["x", "out"], torch.bfloat16)
    _check_dtype([weight, bias], ["weight", "bias"], torch.float32)
    _require(x.dim() == 2 and x.shape == out.shape, "x and out must be [rows, C] of equal shape")
    _require(weight.numel() == x.shape[1] and bias.numel() == x.shape[1], "weight / bias must have C elements")
    st = _cabi.load().f3d_layernorm_bf16(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), x.shape[0], x.shape[1], float(eps),
                                         1 if gelu else 0, _dev_index(dev), _stream(dev))
    _cabi.check(st, "layernorm_bf16")


def layernorm_bwd_bf16(x, grad_out, weight, grad_x, grad_weight, grad_bias, eps=1e-5) -> None:
    """Backward of layernorm_bf16 (without GELU): x, grad_out, grad_x bf16 [rows, C]; weight, grad_weight, grad_bias
    fp32 [C].  Not part of the reference's operator module (its LayerNorm backward comes from TransformerEngine)."""
    dev = _check_tensors([x, grad_out, weight, grad_x, grad_weight, grad_bias], ["x", "grad_out", "weight", "grad_x", "grad_weight", "grad_bias"])
    _check_dtype([x, grad_out, grad_x], ["x", "grad_out", "grad_x"], torch.bfloat16)
    _check_dtype([weight, grad_weight, grad_bias], ["weight", "grad_weight", "grad_bias"], torch.float32)
    _require(x.dim() == 2 and x.shape == grad_out.shape == grad_x.shape, "x, grad_out and grad_x must be [rows, C] of equal shape")
    _require(weight.numel() == x.shape[1] == grad_weight.numel() == grad_bias.numel(), "weight, grad_weight, grad_bias must be [C]")
    st = _cabi.load().f3d_layernorm_bwd_bf16(_ptr(x), _ptr(grad_out), _ptr(weight), _ptr(grad_x), _ptr(grad_weight), _ptr(grad_bias),
                                             x.shape[0], x.shape[1], float(eps), _dev_index(dev), _stream(dev))
    _cabi.check(st, "layernorm_bwd_bf16")


def swiglu_bwd_bf16(pre_act, grad_out, grad_pre_act) -> None:
    """Gradient of silu(gate) * up with respect to pre_act = [gate | up] (bf16 [rows, 2F]); grad_out bf16 [rows, F].
    Not part of the reference's operator module (its MLP backward is TransformerEngine's)."""
    dev = _check_tensors([pre_act, grad_out, grad_pre_act], ["pre_act", "grad_out", "grad_pre_act"])
    _check_dtype([pre_act, grad_out, grad_pre_act], ["pre_act", "grad_out", "grad_pre_act"], torch.bfloat16)
    _require(pre_act.dim() == 2 and grad_out.dim() == 2 and pre_act.shape == grad_pre_act.shape, "pre_act and grad_pre_act must be [rows, 2F]")
    _require(pre_act.shape[0] == grad_out.shape[0] and pre_act.shape[1] == 2 * grad_out.shape[1], "grad_out must be [rows, F]")
    st = _cabi.load().f3d_swiglu_bwd_bf16(_ptr(pre_act), _ptr(grad_out), _ptr(grad_pre_act), pre_act.shape[0], grad_out.shape[1],
                                          _dev_index(dev), _stream(dev))
    _cabi.check(st, "swiglu_bwd_bf16")


def gelu_bwd_bf16(pre_act, grad_out, grad_pre_act, tanh_form: bool = False) -> None:
    """grad_pre_act = grad_out * gelu'(pre_act), all bf16 of one shape: the exact (error function) form, or the tanh form
    of the GEMM's GELU epilogue.  Not part of the reference's operator module (its GELU backward is torch autograd's)."""
    dev = _check_tensors([pre_act, grad_out, grad_pre_act], ["pre_act", "grad_out", "grad_pre_act"])
    _check_dtype([pre_act, grad_out, grad_pre_act], ["pre_act", "grad_out", "grad_pre_act"], torch.bfloat16)
    _require(pre_act.shape == grad_out.shape == grad_pre_act.shape, "pre_act, grad_out and grad_pre_act must have one shape")
    st = _cabi.load().f3d_gelu_bwd_bf16(_ptr(pre_act), _ptr(grad_out), _ptr(grad_pre_act), pre_act.numel(), int(bool(tanh_form)),
                                        _dev_index(dev), _stream(dev))
    _cabi.check(st, "gelu_bwd_bf16")


def colsum_bf16(x, out) -> None:
    """out fp32 [C] = sum over the rows of x bf16 [rows, C] (the bias gradient of a projection), in a fixed order."""
    dev = _check_tensors([x, out], ["x", "out"])
    _check_dtype([x], ["x"], torch.bfloat16)
    _check_dtype([out], ["out"], torch.float32)
    _require(x.dim() == 2 and out.numel() == x.shape[1], "x must be [rows, C] and out [C]")
    st = _cabi.load().f3d_colsum_bf16(_ptr(x), _ptr(out), x.shape[0], x.shape[1], _dev_index(dev), _stream(dev))
    _cabi.check(st, "colsum_bf16")


def coord_embed_bf16(coords, weight, bias, out) -> None:
    """out = coords @ weight.T + bias for fp16 coords [rows, 3], fp32 weight [C, 3] / bias [C], bf16 out [rows, C].
    Not part of the reference's operator module (it embeds with te.Linear, flash3dxfmr/layers/psh_ops.py:62)."""
    dev = _check_tensors([coords, weight, bias, out], ["coords", "weight", "bias", "out"])
    _check_dtype([coords], ["coords"], torch.float16)
    _check_dtype([weight, bias], ["weight", "bias"], torch.float32)
    _check_dtype([out], ["out"], torch.bfloat16)
    _require(coords.dim() == 2 and coords.shape[1] == 3, "coords must be [rows, 3]")
    _require(weight.dim() == 2 and weight.shape[1] == 3 and bias.numel() == weight.shape[0], "weight must be [C, 3], bias [C]")
    _require(out.dim() == 2 and out.shape[0] == coords.shape[0] and out.shape[1] == weight.shape[0], "out must be [rows, C]")
    st = _cabi.load().f3d_coord_embed_bf16(_ptr(coords), _ptr(weight), _ptr(bias), _ptr(out), coords.shape[0], weight.shape[0],
                                           _dev_index(dev), _stream(dev))
    _cabi.check(st, "coord_embed_bf16")


def coord_embed_bwd(coords, grad_out, grad_weight, grad_bias=None) -> None:
    """grad_weight fp32 [C, 3] = grad_out^T coords, grad_bias fp32 [C] = column sums of grad_out, for fp16 coords [rows, 3]
    and bf16 grad_out [rows, C]; fixed summation order.  Not part of the reference's operator module."""
    ts = [coords, grad_out, grad_weight] + ([grad_bias] if grad_bias is not None else [])
    dev = _check_tensors(ts, ["coords", "grad_out", "grad_weight", "grad_bias"][:len(ts)])
    _check_dtype([coords], ["coords"], torch.float16)
    _check_dtype([grad_out], ["grad_out"], torch.bfloat16)
    _check_dtype(ts[2:], ["grad_weight", "grad_bias"][:len(ts) - 2], torch.float32)
    _require(coords.dim() == 2 and coords.shape[1] == 3 and grad_out.dim() == 2 and grad_out.shape[0] == coords.shape[0],
             "coords must be [rows, 3] and grad_out [rows, C]")
    _require(tuple(grad_weight.shape) == (grad_out.shape[1], 3), "grad_weight must be [C, 3]")
    _require(grad_bias is None or grad_bias.numel() == grad_out.shape[1], "grad_bias must be [C]")
    st = _cabi.load().f3d_coord_embed_bwd(_ptr(coords), _ptr(grad_out), _ptr(grad_weight), _ptr(grad_bias) if grad_bias is not None else None,
                                          coords.shape[0], grad_out.shape[1], _dev_index(dev), _stream(dev))
    _cabi.check(st, "coord_embed_bwd")


def collate_points_f32(records, coords, extra=None) -> None:
    """records fp32 [rows, dim] (x, y, z, further channels) -> coords fp16 [rows, 3] and extra fp32 [rows, dim - 3]:
    the cast and slice of collate_coords_flat_sep (flash3dxfmr/psh/batching.py:13-28) in one pass on the device."""
    ts = [records, coords] + ([extra] if extra is not None else [])
    dev = _check_tensors(ts, ["records", "coords", "extra"][:len(ts)])
    _check_dtype([records], ["records"], torch.float32)
    _check_dtype([coords], ["coords"], torch.float16)
    _require(records.dim() == 2 and tuple(coords.shape) == (records.shape[0], 3), "records must be [rows, dim], coords [rows, 3]")
    if extra is not None:
        _check_dtype([extra], ["extra"], torch.float32)
        _require(records.shape[1] > 3 and tuple(extra.shape) == (records.shape[0], records.shape[1] - 3),
                 "extra must be [rows, dim - 3]")
    st = _cabi.load().f3d_collate_points_f32(_ptr(records), _ptr(coords), _ptr(extra) if extra is not None else None,
                                             records.shape[0], records.shape[1], _dev_index(dev), _stream(dev))
    _cabi.check(st, "collate_points_f32")


def scatter_index(bucket_id, bucket_offset, cumsum_counter, batch_sep, out2in, in2out=None) -> None:
    """out2in[row in bucket order] = input row (rows past the input length get len + 3, the padding mark of
    batch_psh_cumsum_scatter_feat_index_postpad_ker, src/psh/batch_psh_bucket.cuh:667) and, when given,
    in2out[input row] = row in bucket order, from the outputs of batch_psh_scatter.  The reference declares the
    operator that would fill scatter_idx_out2in but never binds it."""
    ts = [bucket_id, bucket_offset, cumsum_counter, batch_sep, out2in] + ([in2out] if in2out is not None else [])
    dev = _check_tensors(ts, ["bucket_id", "bucket_offset", "cumsum_counter", "batch_sep", "out2in", "in2out"][:len(ts)])
    _check_dtype([bucket_id], ["bucket_id"], torch.uint16)
    _check_dtype(ts[1:], ["bucket_offset", "cumsum_counter", "batch_sep", "out2in", "in2out"][:len(ts) - 1], torch.uint32)
    n = bucket_id.numel()
    _require(bucket_offset.numel() == n, "bucket_offset must have one entry per point")
    _require(cumsum_counter.dim() == 2 and cumsum_counter.shape[0] == batch_sep.numel(), "cumsum_counter must be [B, num_bucket]")
    _require(out2in.numel() >= n, "out2in must hold at least one entry per point")
    _require(in2out is None or in2out.numel() == n, "in2out must have one entry per point")
    st = _cabi.load().f3d_scatter_index(_ptr(bucket_id), _ptr(bucket_offset), _ptr(cumsum_counter), _ptr(batch_sep), _ptr(out2in),
                                        _ptr(in2out) if in2out is not None else None, n, batch_sep.numel(),
                                        cumsum_counter.shape[1], out2in.numel(), _dev_index(dev), _stream(dev))
    _cabi.check(st, "scatter_index")


def gather_rows(src, index, out) -> None:
    """out[i] = src[index[i]] over rows of any element type; rows whose index is not a row of src are zero."""
    dev = _check_tensors([src, index, out], ["src", "index", "out"])
    _check_dtype([index], ["index"], torch.uint32)
    _require(src.dim() == 2 and out.dim() == 2 and src.shape[1] == out.shape[1] and src.dtype == out.dtype,
             "src and out must be [rows, C] of one dtype and width")
    _require(index.numel() == out.shape[0], "index must have one entry per row of out")
    st = _cabi.load().f3d_gather_rows(_ptr(src), _ptr(index), _ptr(out), out.shape[0], src.shape[0],
                                      src.shape[1] * src.element_size(), _dev_index(dev), _stream(dev))
    _cabi.check(st, "gather_rows")


def launch_count() -> int:
    """Kernels launched by the native library since it was loaded."""
    return int(_cabi.load().f3d_launch_count())


def batch_psh_scatter_pad_hash_noalloc(coord, bucket_id, bucket_counter, bucket_offset, batch_sep, instance_max_N,
                                       num_bucket, bucket_divisor, bucket_size, num_vox, bbox_min, bbox_max,
                                       probe_offsets, cumsum_counter, scatter_coord, pad_num, hash_type) -> None:
    """batch_psh_scatter_pad_hash for hosts that may not allocate device memory: same arguments and results, but
    the library's scratch tables sit in a fixed 4 MiB device array instead of a cudaMalloc'ed workspace.  Use it
    when the process's GPU memory is owned by another allocator or when cudaMalloc's device-wide synchronisation
    is not acceptable.  Batches whose tables do not fit raise RuntimeError; calls must not overlap on one GPU; the
    first call on a device should be made outside stream capture.  No counterpart in the reference."""
    tensors = [coord, bucket_id, bucket_counter, bucket_offset, batch_sep, probe_offsets, cumsum_counter,
               scatter_coord, bbox_min, bbox_max]
    names = ["coord", "bucket_id", "bucket_counter", "bucket_offset", "batch_sep", "probe_offsets", "cumsum_counter",
             "scatter_coord", "bbox_min", "bbox_max"]
    dev = _check_tensors(tensors, names)
    _check_dtype([coord, scatter_coord, bbox_min, bbox_max], ["coord", "scatter_coord", "bbox_min", "bbox_max"],
                 torch.float16)
    _check_dtype([bucket_counter, bucket_offset, batch_sep, cumsum_counter],
                 ["bucket_counter", "bucket_offset", "batch_sep", "cumsum_counter"], torch.uint32)
    _check_dtype([bucket_id], ["bucket_id"], torch.uint16)
    _check_dtype([probe_offsets], ["probe_offsets"], torch.int16)
    _require(coord.dim() == 2 and coord.shape[1] == 3 and scatter_coord.dim() == 2 and scatter_coord.shape[1] == 3,
             "coord and scatter_coord must be [rows, 3]")
    total_n, batch = coord.shape[0], batch_sep.shape[0]
    _require(bucket_id.numel() >= total_n and bucket_offset.numel() >= total_n,
             "bucket_id / bucket_offset are shorter than coord")
    _require(bucket_counter.numel() == batch * num_bucket and cumsum_counter.numel() == batch * num_bucket,
             f"bucket_counter / cumsum_counter must be [{batch},{num_bucket}]")
    _require(probe_offsets.numel() == 128 * 3 and bbox_min.numel() == 3 and bbox_max.numel() == 3,
             "probe_offsets must be [128,3] and the bounding box 3 + 3 values")
    st = _cabi.load().f3d_batch_psh_scatter_pad_hash_noalloc(
        _ptr(coord), _ptr(bucket_id), _ptr(bucket_counter), _ptr(bucket_offset), _ptr(batch_sep),
        total_n, batch, int(instance_max_N), int(num_bucket), int(bucket_divisor), int(bucket_size), int(num_vox),
        _ptr(bbox_min), _ptr(bbox_max), _ptr(probe_offsets), _ptr(cumsum_counter), _ptr(scatter_coord),
        scatter_coord.shape[0], float(pad_num), int(hash_type), _dev_index(dev), _stream(dev))
    _cabi.check(st, "batch_psh_scatter_pad_hash_noalloc")


def buck_swin_bwd(Q, K, V, O, dO, LSE, Delta, dQ, dK, dV, Scope_buckets, bucket_size) -> None:
    """f3d::buck_swin_bwd (declared src/f3d_frontend.cu:94-97; caller flash3dxfmr/layers/buck_swin.py:91).
    Delta, dQ, dK, dV are written in place."""
    dev, (b, l, h, d) = _check_qkv([Q, K, V, O, dO, dQ, dK, dV], ["Q", "K", "V", "O", "dO", "dQ", "dK", "dV"])
    _check_tensors([LSE, Delta, Scope_buckets], ["LSE", "Delta", "Scope_buckets"])
    _check_dtype([LSE, Delta], ["LSE", "Delta"], torch.float32)
    _check_dtype([Scope_buckets], ["Scope_buckets"], torch.uint32)
    _require(tuple(LSE.shape) == (b, l, h) and tuple(Delta.shape) == (b, l, h), f"LSE and Delta must be [{b},{l},{h}]")
    _require(Scope_buckets.dim() == 2, "Scope_buckets must be [num_scopes, scope_size]")
    st = _cabi.load().f3d_buck_swin_bwd(_ptr(Q), _ptr(K), _ptr(V), _ptr(O), _ptr(dO), _ptr(LSE), _ptr(Delta), _ptr(dQ),
                                        _ptr(dK), _ptr(dV), _ptr(Scope_buckets), b, l, h, d, Scope_buckets.shape[0],
                                        Scope_buckets.shape[1], int(bucket_size), _dev_index(dev), _stream(dev))
    _cabi.check(st, "buck_swin_bwd")
