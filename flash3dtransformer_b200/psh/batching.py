"""Flat batching helpers (reference: flash3dxfmr/psh/batching.py:13-47).  A batch of scenes is one [N, 3] tensor
plus `seps`, the inclusive end row of every scene."""
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


def sep2sizes(seps: torch.Tensor) -> torch.Tensor:
    wide = seps.to(torch.int64)
    sizes = torch.diff(wide, prepend=wide.new_zeros(1))
    return sizes.to(seps.dtype)


def max_inslen_from_seps(seps: torch.Tensor) -> int:
    return int(sep2sizes(seps.to(torch.int64)).max())


def bulk_to(ts: List[torch.Tensor], dest):
    return [t.to(dest) for t in ts]


def cdiv_int(a: torch.Tensor, b):
    return (a + (b - 1)) / b
