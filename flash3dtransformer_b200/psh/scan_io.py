"""Raw LiDAR scans to operator inputs.

Scan files of the KITTI / nuScenes kind are flat arrays of fp32 records, one per point: x, y, z, intensity (KITTI, four
floats) plus a ring index (nuScenes, five floats).  The reference reads them with numpy and leaves cast, slice and
concatenation to torch on the host (tests/test_psh.py:31-44, flash3dxfmr/psh/batching.py:13-28).  Here the files of a
batch are read into ONE pinned host buffer, copied to the device once, and a single kernel produces the fp16
coordinates and the remaining channels (lib.pshattn.collate_points_f32).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..lib import pshattn
from . import batching


def read_scan_bins(paths: Sequence[str], point_dim: int = 4, pin: bool = True) -> Tuple[torch.Tensor, List[int]]:
    """Read scan files into one fp32 [sum N_i, point_dim] host tensor (pinned when a GPU is present) and return it with
    the number of points of every file.  A file whose size is not a whole number of records raises ValueError."""
    if point_dim < 3:
        raise ValueError(f"a point record needs at least x, y, z (got point_dim={point_dim})")
    rec_bytes = 4 * point_dim
    sizes = []
    for p in paths:
        nbytes = os.path.getsize(p)
        if nbytes % rec_bytes:
            raise ValueError(f"{p}: {nbytes} bytes is not a whole number of {point_dim}-float records")
        sizes.append(nbytes // rec_bytes)
    total = sum(sizes)
    host = torch.empty(total, point_dim, dtype=torch.float32, pin_memory=bool(pin and torch.cuda.is_available()))
    flat = host.numpy().reshape(-1)
    row = 0
    for p, n in zip(paths, sizes):
        if n:
            with open(p, "rb") as f:
                got = f.readinto(memoryview(flat[row * point_dim:(row + n) * point_dim]).cast("B"))
            if got != n * rec_bytes:
                raise ValueError(f"{p}: short read ({got} of {n * rec_bytes} bytes)")
        row += n
    return host, sizes


def collate_scans(records: torch.Tensor, sizes: Sequence[int], device, want_extra: bool = True):
    """records fp32 [N, dim] (host or device) and per-scene point counts -> (coords fp16 [N, 3], extra fp32 [N, dim - 3]
    or None, seps uint32 [B]) on `device`: what collate_coords_flat_sep (flash3dxfmr/psh/batching.py:13-28) returns for
    coord_dtype=float16, sep_dtype=uint32, plus the channels it drops.  The separators carry their host copy, so the
    layers never read them back."""
    if records.dim() != 2 or records.dtype != torch.float32 or records.shape[1] < 3:
        raise RuntimeError(f"records must be fp32 [N, >=3], got {records.dtype} {tuple(records.shape)}")
    n = records.shape[0]
    if sum(int(s) for s in sizes) != n:
        raise RuntimeError(f"scene sizes add up to {sum(int(s) for s in sizes)}, records hold {n} points")
    device = torch.device(device)
    dev_rec = records.to(device, non_blocking=True).contiguous()
    coords = torch.empty(n, 3, dtype=torch.float16, device=device)
    extra = None
    if want_extra and records.shape[1] > 3:
        extra = torch.empty(n, records.shape[1] - 3, dtype=torch.float32, device=device)
    pshattn.collate_points_f32(dev_rec, coords, extra)
    seps_cpu = torch.cumsum(torch.tensor([int(s) for s in sizes], dtype=torch.int64), dim=0)
    seps = batching.attach_host_seps(seps_cpu.to(torch.uint32).to(device), seps_cpu)
    return coords, extra, seps


def load_scans(paths: Sequence[str], device, point_dim: int = 4, want_extra: bool = True):
    """Files -> (coords fp16 [N, 3], extra fp32 [N, point_dim - 3] or None, seps uint32 [B]) on `device`."""
    records, sizes = read_scan_bins(paths, point_dim)
    return collate_scans(records, sizes, device, want_extra)
