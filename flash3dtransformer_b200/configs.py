"""Model configurations of the benchmark workloads, expressed with the reference's own spec dataclasses
(F3DLevelSpecs / XFMRSpecs, flash3dxfmr/layers/flash3d.py:51-60, stage.py:21-28).  The layout mirrors the
reference's whole-model test (tests/test_psh_hourglass.py:51-163): bucket 512, scope 8, pooled lengths aligned to
bucket*scope, hidden width 4*C, heads = C/32."""
from __future__ import annotations

from functools import partial
from typing import Sequence

from torch import nn

from . import layers
from .psh import bucket_scope


def hourglass_specs(channels: Sequence[int], depths: Sequence[int], bucket_size: int = 512, scope_size: int = 8,
                    head_dim: int = 32, reduction_op="mean"):
    """Encoder stages with the given channels/depths and a mirrored decoder."""
    plan = lambda i: bucket_scope.SwinPlan("swin", bucket_size, scope_size, i)
    norm = partial(nn.LayerNorm, eps=1e-5)
    levels = []
    for c, d in zip(channels, depths):
        blocks = [layers.XFMRSpecs(channels=c, hid_channels=4 * c, num_heads=max(1, c // head_dim), qkv_bias=True,
                                   swin_plan=plan(i), norm_layer=norm) for i in range(d)]
        levels.append(layers.F3DLevelSpecs(
            encoder_specs=list(blocks), decoder_specs=list(blocks), reduction_op=reduction_op,
            pool_align=bucket_scope.swinable_alignment(bucket_size, scope_size),
            pool_norm=norm, pool_act=nn.GELU, unpool_norm=norm, unpool_act=nn.GELU))
    return levels


def flash3d_backbone(channels=(32, 64, 128, 256, 512), depths=(2, 2, 2, 6, 2), bucket_size: int = 512,
                     scope_size: int = 8, hash_op: int = 2, scatter_input_feat: bool = False,
                     restore_input_order: bool = False):
    """The 5-stage hourglass backbone: channels 32/64/128/256/512, depths 2/2/2/6/2, stride-2 pooling between
    stages, mirrored decoder with additive unpooling."""
    return layers.Flash3D(hourglass_specs(channels, depths, bucket_size, scope_size), bucket_size, scope_size, hash_op,
                          scatter_input_feat=scatter_input_feat, restore_input_order=restore_input_order)
