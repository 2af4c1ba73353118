"""PSH scatter layers (mirror of the reference's flash3dxfmr/layers/psh_ops.py:16-67)."""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn

from ..psh import arithmatic as f3darith
from ..psh import psh_main as pm
from .functional import CoordEmbedFn


class PSHScatterLayer(nn.Module):
    def __init__(self, bucket_size: int = 512) -> None:
        super().__init__()
        self.bucket_size = bucket_size

    def forward(self, coords, seps, hash_op: int) -> Tuple[torch.Tensor, pm.BucketScatterBuffers]:
        pad_to = f3darith.cdiv(coords.shape[0], self.bucket_size) * self.bucket_size
        return pm.batch_bucket_scatter(coords, seps, self.bucket_size, pad_to, hash_op)


class PSH3DCoordEmbedding(nn.Module):
    """Bucket-sorts the coordinates and embeds them with a 3 -> C linear layer (the reference uses te.Linear,
    psh_ops.py:61).  `bbox` optionally carries the bounding box of the global batch for scene-sharded runs."""

    def __init__(self, emb_dim: int, bucket_size, alignment, feat_dtype=torch.bfloat16):
        super().__init__()
        self.bucket_size = bucket_size
        self.alignment = alignment
        self.feat_dtype = feat_dtype
        self.lin = nn.Linear(3, emb_dim)

    def forward(self, coords, seps, hash_op, bbox=None, mean_n=None, scene_base=None, want_index=False):
        """Embedded features [pad_to, C] in bucket order; with `want_index` also (out2in, in2out) of the scatter."""
        pad_to = f3darith.cdiv(coords.shape[0], self.alignment) * self.alignment
        scattered, buffers = pm.batch_bucket_scatter(coords, seps, self.bucket_size, pad_to, hash_op, bbox=bbox, mean_n=mean_n,
                                                scene_base=scene_base)
        # K = 3 is not a tensor-core GEMM: the embedding kernel does the three FMAs per output
        out = CoordEmbedFn.apply(scattered if scattered.dtype == torch.float16 else scattered.to(torch.float16),
                                 self.lin.weight, self.lin.bias)
        out = out if self.feat_dtype == torch.bfloat16 else out.to(self.feat_dtype)
        if want_index:
            return out, pm.scatter_index(buffers, seps, pad_to)
        return out
