"""Transformer block and stage (mirror of the reference's flash3dxfmr/layers/stage.py:21-197).

XFMR keeps the reference's dataflow x -> norm -> attention -> + x -> MLP(with its own LayerNorm) -> + (stage.py:
90-101); the two residual additions are fused into the epilogues of the output projection and of the MLP's second
GEMM.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.cuda.nvtx as nvtx
from torch import nn

from . import buck_swin, elem_wise
from . import functional as F3
from ..psh import bucket_scope
from ..psh import dev_context as f3ddev


@dataclass(slots=True)
class XFMRSpecs:
    channels: int
    hid_channels: int
    num_heads: int
    qkv_bias: bool
    swin_plan: bucket_scope.SwinPlan
    norm_layer: callable


class XFMR(nn.Module):
    NVTX_SCOPE = "XFMR"

    def __init__(self, channels: int, hid_chann: int, num_heads: int, buck_size: int, qkv_bias: bool,
                 swin_plan: bucket_scope.SwinPlan, norm_layer: callable):
        super().__init__()
        self.set_chnn = channels
        self.swin_plan = swin_plan
        self.norm = norm_layer(channels)
        self.bwa = buck_swin.BucketSwinAttentionModule(channels, num_heads, buck_size, qkv_bias)
        self.mlp = elem_wise.MLP(channels, hid_chann)

    def forward(self, reduced_coord, reduced_feat, reduced_sep):
        """(coords, features [N, C], seps) -> features [N, C]; coords and seps are unused, as in the reference."""
        assert reduced_feat.dim() == 2, f"Expect input features have two axes [N, C], but got shape={reduced_feat.shape}"
        n, c = reduced_feat.shape
        assert c == self.set_chnn, f"Expect input feat_dim={self.set_chnn}, but got {c}"
        scope_bucks = self.swin_plan.gen_scopes_from_plan(n, reduced_feat.device)
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        feat = reduced_feat if reduced_feat.dtype == torch.bfloat16 else reduced_feat.to(torch.bfloat16)
        x = F3.apply_norm(self.norm, feat)
        mid = self.bwa(x.view(1, n, c), scope_bucks, residual=feat).view(n, c)
        out = self.mlp(mid, residual=mid)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return out


class Stage(nn.Module):
    """Encoder blocks -> middle submodule -> decoder blocks, all with the (coord, feat, sep) signature."""
    NVTX_SCOPE = "Stage"

    def __init__(self, encoder_specs: List[XFMRSpecs], buck_size: int, submodule: nn.Module,
                 decoder_specs: List[XFMRSpecs]):
        super().__init__()
        if submodule is None:
            raise ValueError("A submodule must be provided for a Stage.")

        def block(spec):
            return XFMR(spec.channels, spec.hid_channels, spec.num_heads, buck_size, spec.qkv_bias, spec.swin_plan,
                        spec.norm_layer)

        self.encoder_blocks = nn.ModuleList([block(s) for s in encoder_specs])
        self.middle = submodule
        self.decoder_blocks = nn.ModuleList([block(s) for s in decoder_specs])

    def forward(self, reduced_coord, reduced_feat, reduced_sep):
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        x = reduced_feat
        for blk in self.encoder_blocks:
            x = blk(reduced_coord, x, reduced_sep)
        x = self.middle(reduced_coord, x, reduced_sep)
        for blk in self.decoder_blocks:
            x = blk(reduced_coord, x, reduced_sep)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return x
