"""Token-wise MLP (mirror of the reference's flash3dxfmr/layers/elem_wise.py:19-33).

The reference wraps TransformerEngine's LayerNormMLP(hidden, ffn, activation="swiglu").  TransformerEngine is not
used here; `LayerNormMLP` below keeps its parameter names (layer_norm_weight/bias, fc1_weight/bias, fc2_weight/bias)
and its structure LN -> Linear(C, 2*ffn) -> silu(first half) * second half -> Linear(ffn, C), with the SwiGLU
fused into the first GEMM's epilogue.
"""
from __future__ import annotations

import math

import torch
import torch.cuda.nvtx as nvtx
from torch import nn

from . import functional as F3
from ..lib import pshattn
from ..psh import dev_context as f3ddev


class LayerNormMLP(nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, activation: str = "swiglu", eps: float = 1e-5):
        super().__init__()
        assert activation in ("swiglu", "gelu"), f"Unsupported activation {activation}"
        self.activation = activation
        self.eps = eps
        fc1_out = 2 * ffn_hidden_size if activation == "swiglu" else ffn_hidden_size
        self.layer_norm_weight = nn.Parameter(torch.ones(hidden_size))
        self.layer_norm_bias = nn.Parameter(torch.zeros(hidden_size))
        self.fc1_weight = nn.Parameter(torch.empty(fc1_out, hidden_size))
        self.fc1_bias = nn.Parameter(torch.zeros(fc1_out))
        self.fc2_weight = nn.Parameter(torch.empty(hidden_size, ffn_hidden_size))
        self.fc2_bias = nn.Parameter(torch.zeros(hidden_size))
        nn.init.normal_(self.fc1_weight, std=0.023)
        nn.init.normal_(self.fc2_weight, std=0.023)

    def forward(self, x: torch.Tensor, residual: torch.Tensor = None) -> torch.Tensor:
        h = F3.layer_norm(x, self.layer_norm_weight, self.layer_norm_bias, self.eps)
        epi = pshattn.EPI_SWIGLU if self.activation == "swiglu" else pshattn.EPI_GELU
        h = F3.linear(h, self.fc1_weight, self.fc1_bias, epilogue=epi)
        return F3.linear(h, self.fc2_weight, self.fc2_bias, residual=residual)


class MLP(nn.Module):
    NVTX_SCOPE = "MLP"

    def __init__(self, in_dim, hidden_dim):
        super().__init__()
        self.mlp = LayerNormMLP(hidden_size=in_dim, ffn_hidden_size=in_dim if hidden_dim is None else hidden_dim,
                                activation="swiglu")

    def forward(self, x, residual=None):
        if f3ddev.get_nvtx():
            nvtx.range_push(self.NVTX_SCOPE)
        res = self.mlp(x, residual)
        if f3ddev.get_nvtx():
            nvtx.range_pop()
        return res
