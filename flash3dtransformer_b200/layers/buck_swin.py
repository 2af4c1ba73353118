"""Bucketed multi-head self-attention layer (mirror of the reference's flash3dxfmr/layers/buck_swin.py:20-197).

Same classes and constructor arguments: BuckSwinFwdFunction, BucketSwinAttention, BucketSwinAttentionModule with
parameters `qkv` (Linear C -> 3C) and `proj` (Linear C -> C).  The QKV projection writes Q, K and V as three
contiguous [L, H, D] tensors straight from the GEMM epilogue, which replaces the reference's chunk + three
.contiguous() copies (buck_swin.py:186-190).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.cuda.nvtx as nvtx
from torch import nn
from torch.autograd import Function

from . import functional as F3
from ..lib import pshattn
from ..psh import dev_context as f3ddev
from ..psh import swin_attn as sa


class BuckSwinFwdFunction(Function):
    """O = windowed softmax attention over the buckets of each scope; backward through buck_swin_bwd."""

    @staticmethod
    def forward(ctx, Q, K, V, scope_buckets, buck_size: int):
        buff = sa.BuckSwinFwdBuffers.create_buckswin_fwd_buff(Q)
        pshattn.buck_swin_fwd(Q, K, V, buff.O, buff.LSE, scope_buckets, buck_size)
        ctx.save_for_backward(Q, K, V, buff.O, buff.LSE)
        ctx.scope_buckets = scope_buckets
        ctx.buck_size = buck_size
        return buff.O

    @staticmethod
    def backward(ctx, grad_output) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, None, None]:
        Q, K, V, O, lse = ctx.saved_tensors
        bwd = sa.BuckSwinBwdBuffers.create_buckswin_buffers(O, ctx.scope_buckets, ctx.buck_size)
        pshattn.buck_swin_bwd(Q, K, V, O, grad_output.contiguous(), lse, bwd.Delta, bwd.dQ, bwd.dK, bwd.dV,
                              ctx.scope_buckets, ctx.buck_size)
        return bwd.dQ, bwd.dK, bwd.dV, None, None


class BuckSwinPackedFunction(Function):
    """The same attention with Q, K and V given as the three [B*L, C] matrices of one packed tensor, the layout the QKV
    projection writes.  The backward hands the three slices of ONE packed gradient to buck_swin_bwd, so autograd neither
    zero-fills a packed gradient per slice nor adds the three up (which cost more HBM traffic than the projection
    itself)."""

    @staticmethod
    def forward(ctx, qkv, shape, scope_buckets, buck_size: int):
        b, l, h, d = shape
        Q, K, V = (qkv[i].view(b, l, h, d) for i in range(3))
        buff = sa.BuckSwinFwdBuffers.create_buckswin_fwd_buff(Q)
        pshattn.buck_swin_fwd(Q, K, V, buff.O, buff.LSE, scope_buckets, buck_size)
        ctx.save_for_backward(qkv, buff.O, buff.LSE)
        ctx.cfg = (shape, scope_buckets, buck_size)
        return buff.O

    @staticmethod
    def backward(ctx, grad_output):
        qkv, O, lse = ctx.saved_tensors
        shape, scope_buckets, buck_size = ctx.cfg
        b, l, h, d = shape
        # scope tables made by SwinPlan are marked when they put every bucket in exactly one scope; then every row of
        # the gradient is written by the kernel and the buffer needs no zero fill
        covered = getattr(scope_buckets, "_f3d_partition_of", -1) == l
        grad = torch.empty_like(qkv) if covered else torch.zeros_like(qkv)
        Q, K, V = (qkv[i].view(b, l, h, d) for i in range(3))
        dQ, dK, dV = (grad[i].view(b, l, h, d) for i in range(3))
        delta = torch.empty(b, l, h, dtype=torch.float32, device=O.device)      # every row is written by the delta kernel
        pshattn.buck_swin_bwd(Q, K, V, O, grad_output.contiguous(), lse, delta, dQ, dK, dV, scope_buckets, buck_size)
        return grad, None, None, None


class BucketSwinAttention(nn.Module):
    def __init__(self, buck_size: int) -> None:
        super().__init__()
        self.buck_size = buck_size

    def forward(self, Q, K, V, scope_buckets):
        assert Q.dim() == 4, f"Expect Q with four axes [B, L, H, D], but got shape={Q.shape}"
        return BuckSwinFwdFunction.apply(Q, K, V, scope_buckets, self.buck_size)


class BucketSwinAttentionModule(nn.Module):
    NVTX_SCOPE = "BucketSwinAttention"

    def __init__(self, channels: int, num_heads: int, buck_size: int, qkv_bias: bool = True):
        super().__init__()
        assert channels % num_heads == 0, f"Channels={channels} NOT divisible by num_heads={num_heads}"
        self.num_heads = num_heads
        self.head_dim = channels // num_heads
        self.qkv = nn.Linear(channels, channels * 3, bias=qkv_bias)
        self.attn = BucketSwinAttention(buck_size)
        self.proj = nn.Linear(channels, channels)

    def forward(self, x: torch.Tensor, scope_buckets: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        """x: [B, L, C] -> [B, L, C].  `residual` ([B*L, C], optional, not in the reference signature) is added in
        the epilogue of the output projection."""
        assert x.dim() == 3, f"Expect input features with three axes [B, L, C], but got shape={x.shape}"
        b, l, c = x.shape
        assert c == self.num_heads * self.head_dim, f"Expect input channels are {self.num_heads * self.head_dim}, but got {c}"
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        qkv = F3.linear(x.reshape(b * l, c), self.qkv.weight, self.qkv.bias, nsplit=3)       # [3, B*L, C]
        attn_out = BuckSwinPackedFunction.apply(qkv, (b, l, self.num_heads, self.head_dim), scope_buckets, self.attn.buck_size)
        out = F3.linear(attn_out.view(b * l, c), self.proj.weight, self.proj.bias, residual=residual).view(b, l, c)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return out
