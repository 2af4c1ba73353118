"""Probe-offset table of the overflow rebalance (reference: flash3dxfmr/psh/bucket.py:19-40)."""
from __future__ import annotations

import itertools
import random

import torch

_CORNERS = [(3, 3, 3), (3, -3, 3), (-3, 3, -3), (-3, -3, -3)]


def probe_offset_rows(shuffle_seed=None):
    """The 128 rows: {-2..2}^3 without the origin (124 rows, x slowest) and four (+-3) corners.  The reference
    shuffles the rows with Python's global RNG on every call (bucket.py:35), which makes the bucket layout differ
    from call to call; here the order is fixed unless a shuffle seed is given."""
    rows = [p for p in itertools.product((-2, -1, 0, 1, 2), repeat=3) if p != (0, 0, 0)] + _CORNERS
    if shuffle_seed is not None:
        random.Random(shuffle_seed).shuffle(rows)
    return rows


_CACHE = {}


def generate_probe_offsets(device, row_major=True, shuffle_seed=None):
    key = (str(device), row_major, shuffle_seed)
    if key not in _CACHE:
        t = torch.tensor(probe_offset_rows(shuffle_seed), dtype=torch.int16)
        if not row_major:
            t = t.transpose(0, 1)
        _CACHE[key] = t.contiguous().to(device)
    return _CACHE[key]
