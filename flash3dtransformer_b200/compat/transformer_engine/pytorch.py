"""`transformer_engine.pytorch` names used by the Flash3D layers, on this library's kernels.

  Linear        flash3dxfmr/layers/psh_ops.py:61 (3 -> C coordinate embedding), layers/flash3d.py (leaf projection)
  LayerNorm     norm_layer of the XFMR blocks in the reference's model test (tests/test_psh_hourglass.py:59)
  LayerNormMLP  flash3dxfmr/layers/elem_wise.py:22-26 (activation "swiglu")

Parameter names follow TransformerEngine (weight / bias; layer_norm_weight, fc1_weight, ...), so state dicts keep
their keys.  There is no CPU path: CPU tensors raise from the operator module.
"""
from __future__ import annotations

import torch
from torch import nn

from flash3dtransformer_b200.layers import functional as F3
from flash3dtransformer_b200.layers.elem_wise import LayerNormMLP  # noqa: F401


class Linear(nn.Linear):
    """y = x W^T + b over the last dimension.  in_features = 3 (coordinates) runs the embedding kernel, every other
    width the tcgen05 GEMM."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if self.in_features == 3 and self.bias is not None:
            y = F3.CoordEmbedFn.apply(x2.to(torch.float16), self.weight, self.bias)
        else:
            y = F3.linear(x2, self.weight, self.bias)
        return y.view(*lead, self.out_features)


class LayerNorm(nn.LayerNorm):
    """LayerNorm over the last dimension on the native kernel (bf16 activations, fp32 statistics)."""

    def __init__(self, hidden_size: int, eps: float = 1e-5, **_ignored):
        super().__init__(hidden_size, eps=eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        y = F3.layer_norm(x.reshape(-1, x.shape[-1]), self.weight, self.bias, self.eps)
        return y.view(*lead, x.shape[-1])
