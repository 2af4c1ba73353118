"""In-bucket pooling layer (mirror of the reference's flash3dxfmr/layers/pooling.py:18-186)."""
from __future__ import annotations

import torch
from torch import nn
from torch.autograd import Function

from ..lib import pshattn
from ..psh import batching as f3dbatch
from ..psh import subbuck as f3dsubbuck

NUM_VOX = 0xFFFF


class SubbuckReduceFunction(Function):
    @staticmethod
    def forward(ctx, coords, input_feat, seps, subbuck_size, reduction_op, out_alignment=1):
        """Returns (reduced_feat, SubbuckBuffers); only reduced_feat is differentiable."""
        max_n = f3dbatch.max_inslen_from_seps(seps)
        feat = input_feat.contiguous()
        sb = f3dsubbuck.SubbuckBuffers.create_subbuck_buff(coords, feat, seps, subbuck_size, out_alignment=out_alignment)
        pshattn.batch_subbuck_reduce(coords, feat, seps, max_n, subbuck_size, NUM_VOX, sb.bbox_min, sb.bbox_max,
                                     sb.subbuck_id, sb.subbuck_off, sb.reduced_sep, sb.reduced_coord, sb.reduced_feat,
                                     sb.unpool_ind, 1, reduction_op)
        ctx.save_for_backward(feat, sb.unpool_ind)
        ctx.subbuck_size = subbuck_size
        ctx.reduction_op = reduction_op
        sb.remove_unused_buffers()
        return sb.reduced_feat, sb

    @staticmethod
    def backward(ctx, grad_reduced_feat, grad_buffers=None):
        input_feat, unpool_ind = ctx.saved_tensors
        grad_input = torch.zeros_like(input_feat)
        pshattn.batch_subbuck_reduce_backward(grad_reduced_feat.contiguous(), input_feat, unpool_ind, grad_input,
                                              ctx.subbuck_size, ctx.reduction_op)
        return None, grad_input, None, None, None, None


class InbucketPoolingLayer(nn.Module):
    REDOP_MAP = {"mean": 0, "sum": 1, "min": 2, "max": 3}

    def __init__(self, reduction_op, out_alignment=1024, subbuck_size=2):
        super().__init__()
        self.out_align = out_alignment
        assert subbuck_size == 2, f"Currently only subbuck_size=2 is supported, input is {subbuck_size}"
        if isinstance(reduction_op, str):
            assert reduction_op in self.REDOP_MAP, f"Unsupported reduction op name:{reduction_op}"
            reduction_op = self.REDOP_MAP[reduction_op]
        self.reduction_op = int(reduction_op)
        self.subbuck_size = subbuck_size

    def forward(self, coords, input_feat, seps):
        return SubbuckReduceFunction.apply(coords, input_feat, seps, self.subbuck_size, self.reduction_op, self.out_align)
