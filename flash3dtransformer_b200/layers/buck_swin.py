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
        q, k, v = (qkv[i].view(b, l, self.num_heads, self.head_dim) for i in range(3))
        attn_out = self.attn(q, k, v, scope_buckets)
        out = F3.linear(attn_out.view(b * l, c), self.proj.weight, self.proj.bias, residual=residual).view(b, l, c)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return out
