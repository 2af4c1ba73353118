"""Host side of the PSH scatter: buffer allocation and the call into the operator module.

Mirror of the reference's flash3dxfmr/psh/psh_main.py:21-125 (`BucketScatterBuffers`, `batch_bucket_scatter`):
same names, same argument meaning, same buffer dtypes and fill values.  Differences, all on the host:
  * scene sizes are read once (one device->host copy) instead of three `.item()` round trips
    (psh_main.py:47,101-102);
  * the probe table is fixed (see psh/bucket.py) so that two calls on the same input give the same layout;
  * num_buck is clamped to >= 1 (the reference divides by zero when the mean scene is smaller than a bucket).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Tuple

import torch

from . import arithmatic as f3darith
from . import batching as f3dbatch
from . import bucket as f3dbuck
from . import dev_context as f3ddev
from . import plan as f3dplan
from ..lib import pshattn

NUM_VOX = 0xFFFF


def bucket_plan(seps: torch.Tensor, bucket_size: int, mean_n=None):
    """(mean scene size, largest scene, num_buck, divisor) as psh_main.py:97-104 computes them.  `mean_n` overrides
    the local mean scene size (a scene-sharded run passes the mean over all ranks' scenes)."""
    sizes = f3dbatch.sep2sizes(f3dbatch.host_seps(seps))
    if mean_n is None:
        mean_n = float(sizes.to(torch.float32).mean()) if sizes.numel() else 0.0
    max_n = int(sizes.max()) if sizes.numel() else 0
    num_buck = max(1, f3darith.round_next_two_power(int(mean_n / bucket_size)))
    divisor = int(math.ceil(NUM_VOX / num_buck))
    return mean_n, max_n, num_buck, divisor


@dataclass(slots=True)
class BucketScatterBuffers:
    bucket_id: torch.Tensor
    bucket_cntr: torch.Tensor
    bucket_offs: torch.Tensor
    bucket_cumsum: torch.Tensor
    probe_offs: torch.Tensor
    scattered_coord: torch.Tensor

    @staticmethod
    def create_buffers(coords: torch.Tensor, seps: torch.Tensor, bucket_size: int, pad_to: int, num_buck=None):
        """Allocate every output of the scatter: ids u16 (ones), counters u32 (zeros), offsets u32 (empty),
        cumsum u32 (zeros), probe table i16 [128,3], scattered coords fp16 [pad_to, D] filled with NaN so that a
        row the kernel misses shows up in the reference's "no NaN" check (tests/test_psh.py:117-120)."""
        total_n, d = coords.shape
        dev = coords.device
        if num_buck is None:
            _, _, num_buck, _ = bucket_plan(seps, bucket_size)
        b = seps.shape[0]
        if f3dplan.enabled():
            # inference inside plan.level_buffers(): the kernels write every element of every output, so the buffers
            # are reused from call to call and not filled
            return f3dplan.pooled(("psh", total_n, d, b, num_buck, pad_to, str(dev)), lambda: BucketScatterBuffers(
                bucket_id=torch.empty(total_n, dtype=torch.uint16, device=dev),
                bucket_cntr=torch.empty(b, num_buck, dtype=torch.uint32, device=dev),
                bucket_offs=torch.empty(total_n, dtype=torch.uint32, device=dev),
                bucket_cumsum=torch.empty(b, num_buck, dtype=torch.uint32, device=dev),
                probe_offs=f3dbuck.generate_probe_offsets(dev, row_major=True),
                scattered_coord=torch.empty((pad_to, d), dtype=torch.float16, device=dev)))
        return BucketScatterBuffers(
            bucket_id=torch.ones(total_n, dtype=torch.uint16, device=dev),
            bucket_cntr=torch.zeros(b, num_buck, dtype=torch.uint32, device=dev),
            bucket_offs=torch.empty(total_n, dtype=torch.uint32, device=dev),
            bucket_cumsum=torch.zeros(b, num_buck, dtype=torch.uint32, device=dev),
            probe_offs=f3dbuck.generate_probe_offsets(dev, row_major=True),
            scattered_coord=torch.full((pad_to, d), float("nan"), dtype=torch.float16, device=dev),
        )


def batch_bucket_scatter(coords: torch.Tensor, seps: torch.Tensor, bucket_size: int, pad_to: int, hash_op: int,
                         bbox=None, mean_n=None, scene_base=None) -> Tuple[torch.Tensor, BucketScatterBuffers]:
    """Bucket and scatter a flat batch of fp16 coordinates.

    hash_op: 1 Z-order div, 2 XOR-sum div, 3 Z-order mod, 4 XOR-sum mod.
    bbox: optional (min, max) fp16 [3] tensors; by default the min/max over the whole batch, as in the reference
    (psh_main.py:117-118).  A scene-sharded multi-GPU run passes the bbox of the global batch here so that bucket
    ids do not depend on the sharding.
    Returns (scattered_coord, buffers).
    """
    f3ddev.init_dev(coords.get_device())
    _, max_n, num_buck, divisor = bucket_plan(seps, bucket_size, mean_n)
    buffers = BucketScatterBuffers.create_buffers(coords, seps, bucket_size, pad_to, num_buck)
    if bbox is None:
        bbox_min, bbox_max = torch.aminmax(coords, dim=0)
    else:
        bbox_min, bbox_max = bbox
    if scene_base is not None:
        f3ddev.get_dev_manager().set_scene_base(scene_base)
    pshattn.batch_psh_scatter_pad_hash(
        coords, buffers.bucket_id, buffers.bucket_cntr, buffers.bucket_offs, seps, max_n, num_buck, divisor,
        bucket_size, NUM_VOX, bbox_min.contiguous(), bbox_max.contiguous(), buffers.probe_offs,
        buffers.bucket_cumsum, buffers.scattered_coord, 0.0, hash_op)
    return buffers.scattered_coord, buffers


def scatter_index(buffers: BucketScatterBuffers, seps: torch.Tensor, pad_to: int, inverse: bool = True):
    """(out2in uint32 [pad_to], in2out uint32 [N] or None) for a finished batch_bucket_scatter: out2in[row in bucket
    order] = input row (padding rows hold N + 3, the mark of batch_psh_cumsum_scatter_feat_index_postpad_ker,
    src/psh/batch_psh_bucket.cuh:667), in2out the inverse.  The reference allocates neither: its feature scatter stops
    at the index (batch_psh_bucket.cuh:735)."""
    n = buffers.bucket_id.numel()
    dev = buffers.bucket_id.device
    out2in = torch.empty(pad_to, dtype=torch.uint32, device=dev)
    in2out = torch.empty(n, dtype=torch.uint32, device=dev) if inverse else None
    pshattn.scatter_index(buffers.bucket_id, buffers.bucket_offs, buffers.bucket_cumsum, seps, out2in, in2out)
    return out2in, in2out
