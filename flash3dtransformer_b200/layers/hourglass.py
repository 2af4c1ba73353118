"""Pooling / unpooling wrappers and the hourglass module (mirror of the reference's
flash3dxfmr/layers/hourglass.py:20-294): Linear -> sub-bucket pooling -> norm -> act on the way down, two Linears
(+ norm, act) and the additive unpooling on the way up, a submodule in between."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.cuda.nvtx as nvtx
from torch import nn

from . import functional as F3
from . import pooling, unpool
from ..psh import dev_context as f3ddev
from ..psh import subbuck as f3dsubbuck


class _Linear(nn.Linear):
    """nn.Linear whose forward runs on the tcgen05 GEMM when the shapes allow it."""

    def forward(self, x):
        if x.is_cuda and x.dim() == 2 and self.in_features % 8 == 0 and self.out_features % 8 == 0:
            return F3.linear(x, self.weight, self.bias)
        return super().forward(x)


class PoolingWrapper(nn.Module):
    NVTX_SCOPE = "PoolingWrapper"

    def __init__(self, in_channels: int, out_channels: int, red_op, out_align, norm_layer: callable = None,
                 act_layer: callable = None):
        super().__init__()
        self.proj = _Linear(in_channels, out_channels)
        self.pooling = pooling.InbucketPoolingLayer(red_op, out_alignment=out_align)
        self.norm = norm_layer(out_channels) if norm_layer is not None else None
        self.act = act_layer() if act_layer is not None else None

    def forward(self, coords, input_feat, seps) -> Tuple[torch.Tensor, torch.Tensor, f3dsubbuck.SubbuckBuffers]:
        """-> (reduced_feat [reduced_N, C_out], projected_feat [N, C_out] for the skip path, SubbuckBuffers)"""
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        projected = self.proj(input_feat)
        reduced_feat, subbuffers = self.pooling(coords, projected, seps)
        if self.norm is not None or self.act is not None:
            reduced_feat = F3.apply_norm(self.norm, reduced_feat, self.act)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return reduced_feat, projected, subbuffers


class AdditiveUnpoolingWrapper(nn.Module):
    NVTX_SCOPE = "AdditiveUnpoolingWrapper"

    def __init__(self, in_channels: int, skip_channels: int, out_channels: int, subbuck_size: int = 2,
                 norm_layer: callable = None, act_layer: callable = None):
        super().__init__()
        self.proj = nn.Sequential(_Linear(in_channels, out_channels))
        self.proj_skip = nn.Sequential(_Linear(skip_channels, out_channels))
        if norm_layer is not None:
            self.proj.add_module("norm", norm_layer(out_channels))
            self.proj_skip.add_module("norm", norm_layer(out_channels))
        if act_layer is not None:
            self.proj.add_module("act", act_layer())
            self.proj_skip.add_module("act", act_layer())
        self.unpool = unpool.AdditiveUnpoolLayer(subbuck_size)

    @staticmethod
    def _branch(seq: nn.Sequential, x):
        """Linear -> (norm) -> (act), with LayerNorm + GELU on the fused native kernel."""
        y = seq[0](x)
        norm = getattr(seq, "norm", None)
        act = getattr(seq, "act", None)
        return F3.apply_norm(norm, y, act) if (norm is not None or act is not None) else y

    def forward(self, residual, down, buffers: f3dsubbuck.SubbuckBuffers) -> torch.Tensor:
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        output = self.unpool(self._branch(self.proj_skip, residual), self._branch(self.proj, down), buffers)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return output


class HourglassModule(nn.Module):
    NVTX_SCOPE = "HourglassModule"

    def __init__(self, pooling_in_channels: int, pooling_out_channels: int, pooling_reduction_op,
                 pooling_length_alignment: int, unpooling_in_channels: int, unpooling_out_channels: int,
                 pooling_norm_layer: callable = None, pooling_act_layer: callable = None,
                 unpooling_norm_layer: callable = None, unpooling_act_layer: callable = None,
                 submodule: nn.Module = None):
        super().__init__()
        if submodule is None:
            raise ValueError("A submodule must be provided for HourglassModule.")
        self.pooling = PoolingWrapper(pooling_in_channels, pooling_out_channels, pooling_reduction_op,
                                      pooling_length_alignment, pooling_norm_layer, pooling_act_layer)
        self.unpooling = AdditiveUnpoolingWrapper(unpooling_in_channels, pooling_out_channels, unpooling_out_channels,
                                                  norm_layer=unpooling_norm_layer, act_layer=unpooling_act_layer)
        self.submodule = submodule

    def forward(self, coords, input_feat, seps) -> torch.Tensor:
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        reduced_feat, residual_feat, buffers = self.pooling(coords, input_feat, seps)
        sub_out = self.submodule(buffers.reduced_coord, reduced_feat, buffers.reduced_sep)
        output = self.unpooling(residual_feat, sub_out, buffers)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return output
