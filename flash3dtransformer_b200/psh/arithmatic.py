"""Integer helpers with the names the reference exposes in flash3dxfmr/psh/arithmatic.py:12-29."""
from __future__ import annotations

import math


def round_next_two_power(v: int) -> int:
    """Smallest power of two >= v for v >= 1 (0 for v <= 0, which is what the reference's bit trick yields)."""
    v = int(v)
    if v <= 0:
        return 0
    return 1 << (v - 1).bit_length()


def round_next_multiply(v, base):
    return type(v)(math.ceil(float(v) / base) * base)


def cdiv(a, b) -> int:
    return int(math.ceil(a / b))
