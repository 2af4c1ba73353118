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
        if self._can_fold(feat):
            out = self._forward_folded(feat, reduced_feat, scope_bucks, n, c)
        else:
            x = F3.apply_norm(self.norm, feat)
            mid = self.bwa(x.view(1, n, c), scope_bucks, residual=feat).view(n, c)
            out = self.mlp(mid, residual=mid)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return out

    # Narrowest block that takes the folded path.  Measured per block on 16 x 120k points (LayerNorm kernels + four
    # GEMMs against four fused GEMMs): C = 32 / 64 / 128 lose 57 / 32 / 9 us (their epilogues are bound by instruction
    # issue, and a LayerNorm kernel over narrow rows costs only 45 us), C = 256 / 512 gain 39 / 75 us.
    FOLD_MIN_CHANNELS = 256

    def _can_fold(self, feat) -> bool:
        """Inference on the GPU with an affine nn.LayerNorm in front of the attention and the SwiGLU MLP, on rows wide
        enough for the fold to pay: both LayerNorms fold into the projections that follow them."""
        norm = self.norm
        return (not torch.is_grad_enabled() and feat.is_cuda and feat.shape[1] % 8 == 0 and isinstance(norm, nn.LayerNorm)
                and norm.elementwise_affine and norm.bias is not None and tuple(norm.normalized_shape) == (feat.shape[1],)
                and self.mlp.mlp.activation == "swiglu" and self.FOLD_MIN_CHANNELS <= feat.shape[1] <= 2048)

    def _forward_folded(self, feat, given, scope_bucks, n, c):
        """LN -> QKV, attention, proj + residual, LN -> fc1 (SwiGLU), fc2 + residual as four GEMMs and the attention
        kernel: no LayerNorm kernel runs.  Each LayerNorm is applied in the epilogue of the projection behind it from the
        row sums that the projection in front of it accumulated; the sums of this block's output travel with the
        returned tensor to the next block, and only a block whose input came from elsewhere (embedding, pooling,
        unpooling) computes them with a pass of its own."""
        stats = getattr(given, "_f3d_row_stats", None)
        if stats is None or stats.shape[0] != n:
            stats = F3.row_stats(feat)
        bwa, m = self.bwa, self.mlp.mlp
        qkv = F3.linear_inference(feat, bwa.qkv.weight, bwa.qkv.bias, nsplit=3, ln=(self.norm.weight, self.norm.bias, self.norm.eps),
                                  ln_stats=stats)
        attn_out = buck_swin.BuckSwinPackedFunction.apply(qkv, (1, n, bwa.num_heads, bwa.head_dim), scope_bucks, bwa.attn.buck_size)
        mid, mid_stats = F3.linear_inference(attn_out.view(n, c), bwa.proj.weight, bwa.proj.bias, residual=feat, want_stats=True)
        h = F3.linear_inference(mid, m.fc1_weight, m.fc1_bias, epilogue=F3.pshattn.EPI_SWIGLU,
                                ln=(m.layer_norm_weight, m.layer_norm_bias, m.eps), ln_stats=mid_stats)
        out, out_stats = F3.linear_inference(h, m.fc2_weight, m.fc2_bias, residual=mid, want_stats=True)
        out._f3d_row_stats = out_stats
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
