"""Flat batching helpers (reference: flash3dxfmr/psh/batching.py:13-47).  A batch of scenes is one [N, 3] tensor
plus `seps`, the cumulative point count after every scene (scene s covers rows [seps[s-1], seps[s]))."""
from __future__ import annotations

from typing import List

import torch


def collate_coords_flat_sep(coords: List[torch.Tensor], coord_dtype=None, sep_dtype=None):
    """[[N_1, D], ..., [N_B, D]] -> (coords [sum N_i, 3] contiguous, seps [B])."""
    flat = torch.cat(coords, dim=0)
    seps = torch.cumsum(torch.tensor([c.shape[0] for c in coords], dtype=torch.int32), dim=-1)
    if coord_dtype is not None:
        flat = flat.to(coord_dtype)
    if sep_dtype is not None:
        seps = seps.to(sep_dtype)
    return flat[:, :3].contiguous(), seps


def host_seps(seps: torch.Tensor) -> torch.Tensor:
    """int64 CPU copy of a separator tensor.  The copy is cached on the tensor object, so a batch costs one
    device-to-host transfer no matter how many layers ask for scene sizes (the reference issues several .item()
    round trips per layer: flash3dxfmr/psh/psh_main.py:47,101-102, flash3dxfmr/layers/pooling.py:45)."""
    cached = getattr(seps, "_f3d_host", None)
    if cached is None:
        cached = seps.detach().to("cpu", torch.int64)
        try:
            seps._f3d_host = cached
        except AttributeError:
            pass
    return cached


def attach_host_seps(seps_dev: torch.Tensor, seps_cpu: torch.Tensor) -> torch.Tensor:
    seps_dev._f3d_host = seps_cpu.to(torch.int64)
    return seps_dev


def sep2sizes(seps: torch.Tensor) -> torch.Tensor:
    wide = seps.to(torch.int64)
    sizes = torch.diff(wide, prepend=wide.new_zeros(1))
    return sizes.to(seps.dtype)


def max_inslen_from_seps(seps: torch.Tensor) -> int:
    return int(sep2sizes(host_seps(seps)).max())


def bulk_to(ts: List[torch.Tensor], dest):
    return [t.to(dest) for t in ts]


def cdiv_int(a: torch.Tensor, b):
    return (a + (b - 1)) / b
