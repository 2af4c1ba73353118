"""CPU oracle of the whole Flash3D backbone forward, composed from the per-operator oracles.
TEST INFRASTRUCTURE ONLY: used by tests/ and by bench.py's cpu_baseline / --impl reference legs; the product path
never imports it.

It walks the same module tree as flash3dtransformer_b200.layers.Flash3D (which mirrors the reference's
flash3dxfmr/layers/flash3d.py:79-166, stage.py:90-197, hourglass.py:268-294, buck_swin.py:165-197,
elem_wise.py:19-33) but reads only the modules' parameters and hyper-parameters and computes every step with the
numpy / torch-CPU oracles in fp32, rounding activations to bf16 wherever the GPU path stores bf16.

Parity status: inherits the status of the operator oracles (PSH hash and sub-bucket partition unpinned beyond the
reference's invariants; attention, pooling and scope tables pinned by golden fixtures).  The MLP follows
TransformerEngine's LayerNormMLP(activation="swiglu") as the reference configures it (elem_wise.py:22-26);
TransformerEngine's source is not part of the reference checkout, so its numerics are PARITY UNPINNED.
"""
from __future__ import annotations

import numpy as np
import torch

from . import attn_oracle as ao
from . import pool_oracle as pl
from . import psh_oracle as po


def _bf(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def _ln(x, w, b, eps, gelu=False):
    y = torch.nn.functional.layer_norm(x, (x.shape[-1],), w.float(), b.float(), eps)
    if gelu:
        y = torch.nn.functional.gelu(y)
    return _bf(y)


def _lin(x, lin, residual=None):
    y = x @ _bf(lin.weight.detach().float()).t()
    if lin.bias is not None:
        y = y + lin.bias.detach().float()
    if residual is not None:
        y = y + residual
    return _bf(y)


def _norm_act(norm, act, x):
    assert isinstance(norm, torch.nn.LayerNorm), "the oracle covers LayerNorm wrappers only"
    assert act is None or isinstance(act, torch.nn.GELU)
    return _ln(x, norm.weight.detach(), norm.bias.detach(), norm.eps, gelu=act is not None)


def xfmr(blk, feat: torch.Tensor) -> torch.Tensor:
    n, c = feat.shape
    scopes = torch.tensor(blk.swin_plan.scope_list(n), dtype=torch.int64)
    x = _norm_act(blk.norm, None, feat)
    bwa = blk.bwa
    qkv = _lin(x, bwa.qkv)
    q, k, v = (t.reshape(1, n, bwa.num_heads, bwa.head_dim) for t in qkv.chunk(3, dim=-1))
    o, _ = ao.buck_swin_fwd(q, k, v, scopes, blk.swin_plan.buck_size)
    mid = _lin(_bf(o).reshape(n, c), bwa.proj, residual=feat)
    m = blk.mlp.mlp
    h = _ln(mid, m.layer_norm_weight.detach(), m.layer_norm_bias.detach(), m.eps)
    y = h @ _bf(m.fc1_weight.detach().float()).t() + m.fc1_bias.detach().float()
    f = y.shape[1] // 2
    h = _bf(torch.nn.functional.silu(y[:, :f]) * y[:, f:])
    out = h @ _bf(m.fc2_weight.detach().float()).t() + m.fc2_bias.detach().float() + mid
    return _bf(out)


def stage(st, coords16: np.ndarray, feat: torch.Tensor, seps: np.ndarray) -> torch.Tensor:
    x = feat
    for blk in st.encoder_blocks:
        x = xfmr(blk, x)
    x = middle(st.middle, coords16, x, seps)
    for blk in st.decoder_blocks:
        x = xfmr(blk, x)
    return x


def middle(mod, coords16, feat, seps):
    if hasattr(mod, "pooling"):          # HourglassModule
        pw, uw = mod.pooling, mod.unpooling
        projected = _lin(feat, pw.proj)
        S = pw.pooling.subbuck_size
        n = coords16.shape[0]
        red_len, _, red_sep = pl.calc_red_sep_sizes(seps, S)
        aligned = -(-red_len // pw.pooling.out_align) * pw.pooling.out_align
        _, _, unpool, rcoord, _ = pl.subbuck_build(coords16, seps, S, red_rows_aligned=aligned)
        red = torch.from_numpy(pl.pool_reduce(projected.numpy(), unpool, n, pw.pooling.reduction_op, aligned, "bf16"))
        red = _norm_act(pw.norm, pw.act, red)
        sub = stage(mod.submodule, rcoord[:red_len], red, red_sep)
        down = _norm_act(getattr(uw.proj, "norm", None), getattr(uw.proj, "act", None), _lin(sub, uw.proj[0]))
        skip = _norm_act(getattr(uw.proj_skip, "norm", None), getattr(uw.proj_skip, "act", None), _lin(projected, uw.proj_skip[0]))
        up = pl.unpool_add(skip.numpy(), down.numpy(), unpool, "bf16")
        return torch.from_numpy(up)
    return _lin(feat, mod.proj)           # LeafModule


def flash3d_forward(model, coords16: np.ndarray, seps: np.ndarray, seed: int = 3407, bbox=None) -> torch.Tensor:
    """coords fp16 [N,3] (numpy), seps [B] -> features [pad_to, C] fp32 (values on the bf16 grid)."""
    with torch.no_grad():
        emb = model.psh_scatter
        sizes = np.diff(np.concatenate([[0], np.asarray(seps, dtype=np.int64)]))
        nb, div = po.psh_params(sizes, emb.bucket_size)
        n = coords16.shape[0]
        pad_to = -(-n // emb.alignment) * emb.alignment
        lo, hi = (coords16.min(0), coords16.max(0)) if bbox is None else bbox
        sc = po.psh_scatter(coords16, seps, nb, div, emb.bucket_size, 0xFFFF, lo, hi, po.probe_table(), pad_to, 0.0,
                            model.first_hashtype, seed)["scattered_coord"]
        x = _bf(torch.from_numpy(sc.astype(np.float32)))
        feat = _bf(x @ _bf(emb.lin.weight.detach().float()).t() + _bf(emb.lin.bias.detach().float()))
        return stage(model.module_tree, coords16, feat, np.asarray(seps, dtype=np.int64))
