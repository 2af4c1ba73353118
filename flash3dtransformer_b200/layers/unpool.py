"""Additive unpooling layer (mirror of the reference's flash3dxfmr/layers/unpool.py:18-105)."""
from __future__ import annotations

from typing import Tuple

import torch
from torch import nn
from torch.autograd import Function

from ..lib import pshattn
from ..psh.subbuck import SubbuckBuffers, UnpoolBuffers, UnpoolGradients


class AdditiveUnpoolFunction(Function):
    @staticmethod
    def forward(ctx, residual_feat, down_feat, buffers: SubbuckBuffers, subbuck_size: int):
        res = residual_feat.contiguous()
        buf = UnpoolBuffers.create_unpool_buff(res)
        # rows behind the pooled range (tail padding of the level above) are zero-filled, not left uninitialised
        pshattn.additive_unpool_fwd(res, down_feat.contiguous(), buf.up_add_feat, buffers.unpool_ind, subbuck_size,
                                    covered_rows=buffers.pooled_rows or None)
        ctx.subbuck_buffers = buffers
        ctx.subbuck_size = subbuck_size
        return buf.up_add_feat

    @staticmethod
    def backward(ctx, grad_up) -> Tuple[torch.Tensor, torch.Tensor, None, None]:
        buffers = ctx.subbuck_buffers
        g = grad_up.contiguous()
        grads = UnpoolGradients.create_unpool_grad(g, buffers)
        pshattn.additive_unpool_bwd(grads.grad_res, grads.grad_down, g, buffers.unpool_ind, ctx.subbuck_size)
        return grads.grad_res, grads.grad_down, None, None


class AdditiveUnpoolLayer(nn.Module):
    def __init__(self, subbuck_size: int = 2) -> None:
        super().__init__()
        assert subbuck_size == 2, f"Currently only subbuck_size=2 is supported, input is {subbuck_size}"
        self.subbuck_size = subbuck_size

    def forward(self, residual_feat, down_feat, buffers: SubbuckBuffers):
        return AdditiveUnpoolFunction.apply(residual_feat, down_feat, buffers, self.subbuck_size)
