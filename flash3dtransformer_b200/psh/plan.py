"""Pre-planned level buffers for inference.

The reference allocates every intermediate buffer of every level on every call and fills most of them with a value the
kernels then overwrite (flash3dxfmr/psh/psh_main.py:31-67, flash3dxfmr/psh/subbuck.py:64-108,
flash3dxfmr/psh/swin_attn.py:17-22).  Inside `with level_buffers():` the buffer factories of this package hand out the
SAME tensors for the same request (shape signature, device, stream) again, unfilled: a forward pass over a batch whose
scene sizes were seen before allocates nothing for its PSH tables, sub-bucket tables, reduced coordinates / features and
log-sum-exp rows, and launches no fill kernel.  `Flash3D.forward` enters the context when autograd is off; with autograd
on, buffers are saved for the backward pass and must stay private to their call, so nothing is shared.

Tensors handed out here are only valid until the next request with the same key on the same stream: results that a
caller keeps (the model's output features) are never taken from the pool.
"""
from __future__ import annotations

import contextlib
from collections import OrderedDict

import torch

_MAX_ENTRIES = 256
_pool: "OrderedDict[tuple, object]" = OrderedDict()
_enabled = False


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def level_buffers(on: bool = True):
    """Share intermediate level buffers across calls inside this context (single stream of work per key)."""
    global _enabled
    prev = _enabled
    _enabled = bool(on)
    try:
        yield
    finally:
        _enabled = prev


def pooled(key: tuple, factory):
    """factory() on the first request for `key` (on the current device and stream), the same object afterwards."""
    if not _enabled:
        return factory()
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    stream = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0
    full = (dev, stream) + key
    hit = _pool.get(full)
    if hit is not None:
        _pool.move_to_end(full)
        return hit
    obj = factory()
    _pool[full] = obj
    while len(_pool) > _MAX_ENTRIES:
        _pool.popitem(last=False)
    return obj


def clear() -> None:
    _pool.clear()
