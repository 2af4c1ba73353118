"""Top-level Flash3D backbone (mirror of the reference's flash3dxfmr/layers/flash3d.py:22-166): PSH coordinate
embedding followed by a recursive tree of Stage(encoder blocks, Hourglass(next level) or Leaf, decoder blocks)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Union

import torch
import torch.cuda.nvtx as nvtx
from torch import nn

from . import hourglass as f3dhourglass
from . import psh_ops
from . import stage as f3dstage
from ..psh import dev_context as f3ddev
from ..psh import plan as f3dplan
from .functional import GatherRowsFn


class LeafModule(nn.Module):
    """Innermost submodule: one projection of the deepest features (the reference uses te.Linear)."""

    def __init__(self, in_dim, out_dim):
        super().__init__()
        self.proj = f3dhourglass._Linear(in_dim, out_dim)

    def forward(self, reduced_coord, reduced_feat, reduced_sep):
        return self.proj(reduced_feat)


@dataclass(slots=True)
class F3DLevelSpecs:
    encoder_specs: List[f3dstage.XFMRSpecs]
    decoder_specs: List[f3dstage.XFMRSpecs]
    reduction_op: Union[int, str]
    pool_align: int
    pool_norm: callable
    pool_act: callable
    unpool_norm: callable
    unpool_act: callable


class Flash3D(nn.Module):
    NVTX_SCOPE = "Flash3D"

    def __init__(self, level_specs: List[F3DLevelSpecs], buck_size: int, scope_size: int, top_level_hash,
                 scatter_input_feat: bool = False, restore_input_order: bool = False):
        """The last two switches (off by default, which is the reference's behaviour) finish what the reference's
        feature scatter started (src/psh/batch_psh_bucket.cuh:617-753): `scatter_input_feat` brings input_feat [N, C]
        into bucket order and adds it to the coordinate embedding, `restore_input_order` returns [N, C] features in the
        order of the input points instead of [pad_to, C] in bucket order."""
        super().__init__()
        self.scatter_input_feat = scatter_input_feat
        self.restore_input_order = restore_input_order
        f3ddev.set_sync_stream(False)
        emb_chann = level_specs[0].encoder_specs[0].channels
        self.first_hashtype = top_level_hash
        # padded to 6 scopes' worth of tokens so that stride plans 1..3 divide the bucket count
        self.psh_scatter = psh_ops.PSH3DCoordEmbedding(emb_chann, buck_size, buck_size * scope_size * 6)
        self.level_specs = level_specs
        self.buck_size = buck_size
        self.scope_size = scope_size
        self.module_tree = self.build_module(0)

    def build_module(self, level: int) -> nn.Module:
        if level >= len(self.level_specs):
            raise ValueError("Level exceeds level_specs length.")
        spec = self.level_specs[level]
        last_enc, first_dec = spec.encoder_specs[-1], spec.decoder_specs[0]
        if level + 1 >= len(self.level_specs):
            sub = LeafModule(last_enc.channels, first_dec.channels)
        else:
            nxt = self.level_specs[level + 1]
            sub = f3dhourglass.HourglassModule(
                pooling_in_channels=last_enc.channels,
                pooling_out_channels=nxt.encoder_specs[0].channels,
                pooling_reduction_op=spec.reduction_op,
                pooling_length_alignment=spec.pool_align,
                unpooling_in_channels=nxt.decoder_specs[-1].channels,
                unpooling_out_channels=first_dec.channels,
                pooling_norm_layer=spec.pool_norm, pooling_act_layer=spec.pool_act,
                unpooling_norm_layer=spec.unpool_norm, unpooling_act_layer=spec.unpool_act,
                submodule=self.build_module(level + 1))
        return f3dstage.Stage(encoder_specs=spec.encoder_specs, buck_size=self.buck_size, submodule=sub,
                              decoder_specs=spec.decoder_specs)

    def forward(self, coords: torch.Tensor, input_feat: torch.Tensor, seps: torch.Tensor, bbox=None,
                mean_n=None, scene_base=None) -> torch.Tensor:
        """coords fp16 [N, 3], seps uint32 [B] -> features [pad_to, C] in bucket-sorted order.  As in the reference
        (flash3d.py:162-163), input_feat is accepted and not read, and the unscattered coords travel down the tree
        next to the scattered features.  `bbox` / `mean_n` (not in the reference) carry the bounding box and mean scene
        size of the global batch in a scene-sharded run (parallel.global_psh_stats), `scene_base` the global index of the
        shard's first scene."""
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        # without autograd the intermediate buffers of every level come from the per-signature pool (psh/plan.py)
        with f3dplan.level_buffers(not torch.is_grad_enabled() and coords.is_cuda):
            out = self._forward(coords, input_feat, seps, bbox, mean_n, scene_base)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return out

    def _forward(self, coords, input_feat, seps, bbox, mean_n, scene_base):
        if self.scatter_input_feat or self.restore_input_order:
            psh_feat, (out2in, in2out) = self.psh_scatter(coords, seps, self.first_hashtype, bbox=bbox, mean_n=mean_n,
                                                          scene_base=scene_base, want_index=True)
            if self.scatter_input_feat:
                psh_feat = psh_feat + GatherRowsFn.apply(input_feat.to(psh_feat.dtype), out2in, in2out)
        else:
            psh_feat = self.psh_scatter(coords, seps, self.first_hashtype, bbox=bbox, mean_n=mean_n, scene_base=scene_base)
        out = self.module_tree(coords, psh_feat, seps)
        if self.restore_input_order:
            out = GatherRowsFn.apply(out, in2out, out2in)
        return out
