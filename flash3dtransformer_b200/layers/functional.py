"""Autograd glue between torch modules and the native operators.

Forward passes run the hand-written kernels (tcgen05 GEMM with fused bias / residual / SwiGLU epilogues, bucketed
attention, pooling, unpooling).  In the backward passes of the projections the input gradient g W runs on the same
tcgen05 GEMM; the weight gradient g^T x (a reduction over all rows) is a plain library GEMM.  The backward passes of
attention, pooling and unpooling run the native kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch.autograd import Function

from ..lib import pshattn

_BF16_CACHE = {}


def bf16_weight(p: torch.Tensor) -> torch.Tensor:
    """bf16 copy of a parameter, refreshed when the parameter is modified in place (optimizer step)."""
    if p.dtype == torch.bfloat16:
        return p.detach()
    key = id(p)
    hit = _BF16_CACHE.get(key)
    if hit is not None and hit[0] == p._version and hit[1].device == p.device and hit[2] is p:
        return hit[1]
    w = p.detach().to(torch.bfloat16).contiguous()
    _BF16_CACHE[key] = (p._version, w, p)
    return w


def _fp32_param(p: torch.Tensor) -> torch.Tensor:
    """fp32 contiguous view of a parameter (the parameter itself when it already is one)."""
    d = p.detach()
    return d if d.dtype == torch.float32 and d.is_contiguous() else d.float().contiguous()


def _fp32_bias(b: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if b is None:
        return None
    return b.detach() if b.dtype == torch.float32 else b.detach().float()


_FOLD_CACHE = {}


def folded_layernorm(weight, bias, gamma, beta):
    """(W' bf16 [N, K], s fp32 [N], b' fp32 [N]) for LayerNorm(gamma, beta) followed by y = x W^T + b:
    W' = W diag(gamma) rounded to bf16, s = row sums of W' as stored, b' = b + W beta.  Cached until one of the four
    parameters is modified in place."""
    key = (id(weight), id(gamma))
    ver = (weight._version, gamma._version, beta._version, bias._version if bias is not None else -1, weight.device)
    hit = _FOLD_CACHE.get(key)
    if hit is not None and hit[0] == ver and hit[4] is weight:
        return hit[1], hit[2], hit[3]
    with torch.no_grad():
        w32 = weight.detach().float()
        wf = (w32 * gamma.detach().float()[None, :]).to(torch.bfloat16).contiguous()
        s = wf.float().sum(dim=1).contiguous()
        bf = w32 @ beta.detach().float()
        if bias is not None:
            bf = bf + bias.detach().float()
        bf = bf.contiguous()
    _FOLD_CACHE[key] = (ver, wf, s, bf, weight)
    return wf, s, bf


def row_stats(x):
    """fp32 [rows, 2] row sums of a bf16 [rows, C] tensor (for a LayerNorm folded into the next projection)."""
    stats = torch.empty(x.shape[0], 2, dtype=torch.float32, device=x.device)
    pshattn.row_stats_bf16(x, stats)
    return stats


def linear_inference(x, weight, bias, residual=None, nsplit=1, epilogue=pshattn.EPI_NONE, ln=None, ln_stats=None,
                     want_stats=False):
    """Forward-only projection on the fused GEMM.  `ln` = (gamma, beta, eps) folds that LayerNorm of x into the GEMM
    (`ln_stats` = row sums of x).  Returns out, or (out, row sums of out) with `want_stats`."""
    m = x.shape[0]
    if ln is not None:
        w, s, b = folded_layernorm(weight, bias, ln[0], ln[1])
        eps = ln[2]
    else:
        w, s, b, eps = bf16_weight(weight), None, _fp32_bias(bias), 1e-5
    n = w.shape[0]
    out_n = n // 2 if epilogue == pshattn.EPI_SWIGLU else n
    shape = (nsplit, m, out_n // nsplit) if nsplit > 1 else (m, out_n)
    out = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
    stats = torch.empty(m, 2, dtype=torch.float32, device=x.device) if want_stats else None
    pshattn.linear_fused(x, w, b, out, residual=residual, nsplit=nsplit, epilogue=epilogue, ln_stats=ln_stats if ln is not None else None,
                         ln_colsum=s, ln_eps=eps, stats_out=stats)
    return (out, stats) if want_stats else out


class CoordEmbedFn(Function):
    """y = x W^T + b for fp16 coordinates x [rows, 3]: the native embedding kernel (no gradient flows into x)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
        pshattn.coord_embed_bf16(x.contiguous(), weight.detach().float().contiguous(), bias.detach().float().contiguous(), out)
        ctx.save_for_backward(x)
        ctx.dtypes = (weight.dtype, bias.dtype)
        return out

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        gb16 = (g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)).contiguous()
        gw = torch.empty(gb16.shape[1], 3, dtype=torch.float32, device=g.device)
        gb = torch.empty(gb16.shape[1], dtype=torch.float32, device=g.device)
        pshattn.coord_embed_bwd(x.contiguous(), gb16, gw, gb)
        return None, gw.to(ctx.dtypes[0]), gb.to(ctx.dtypes[1])


# Largest weight (elements) whose gradient goes to the native kernel: above it the output tiles outnumber the SMs, the
# operands are re-read once per tile column, and the library's split-K GEMM measured faster (N x K = 4096 x 512: 198
# against 98 us; 2048 x 256 and below: 40-100 us against 48-127 us).
_WGRAD_MAX_ELEMS = 512 * 1024


def _param_grads(g, xb, weight, bias):
    """(grad_weight, grad_bias) of y = x W^T + b for the bf16 gradient g [M, N] and input xb [M, K]: one native pass
    over both (fp32 results, fixed summation order) for the shapes it takes, else a library GEMM plus the native
    column sums."""
    n, k = g.shape[1], xb.shape[1]
    if g.dtype == torch.bfloat16 and pshattn.wgrad_supported(n, k) and n * k <= _WGRAD_MAX_ELEMS:
        gw = torch.empty(n, k, dtype=torch.float32, device=g.device)
        gb = torch.empty(n, dtype=torch.float32, device=g.device) if bias is not None else None
        pshattn.linear_wgrad_bf16(g, xb, gw, gb)
        return gw.to(weight.dtype), (gb.to(bias.dtype) if bias is not None else None)
    gw = (g.t() @ xb).to(weight.dtype)
    gb = None
    if bias is not None:
        if g.dtype == torch.bfloat16 and n % 8 == 0:
            gb32 = torch.empty(n, dtype=torch.float32, device=g.device)
            pshattn.colsum_bf16(g, gb32)
            gb = gb32.to(bias.dtype)
        else:
            gb = g.float().sum(0).to(bias.dtype)
    return gw, gb


class GatherRowsFn(Function):
    """out[i] = src[index[i]] (zero rows where index[i] is the padding mark).  `inverse` maps the rows of src to the
    rows of out, so that the backward is the same gather run through it: with (out2in, in2out) it scatters features into
    bucket order, with (in2out, out2in) it restores the input order."""

    @staticmethod
    def forward(ctx, src, index, inverse):
        out = torch.empty(index.numel(), src.shape[1], dtype=src.dtype, device=src.device)
        pshattn.gather_rows(src.contiguous(), index, out)
        ctx.save_for_backward(inverse)
        return out

    @staticmethod
    def backward(ctx, g):
        (inverse,) = ctx.saved_tensors
        gx = torch.empty(inverse.numel(), g.shape[1], dtype=g.dtype, device=g.device)
        pshattn.gather_rows(g.contiguous(), inverse, gx)
        return gx, None, None


class LinearFn(Function):
    """y = x W^T + b (+ residual); forward on the tcgen05 GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, nsplit, epilogue):
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        xb = xb.contiguous()
        m, n = xb.shape[0], weight.shape[0]
        out_n = n // 2 if epilogue == pshattn.EPI_SWIGLU else n
        shape = (nsplit, m, out_n // nsplit) if nsplit > 1 else (m, out_n)
        out = torch.empty(shape, dtype=torch.bfloat16, device=x.device)
        res = None if residual is None else residual.contiguous()
        pshattn.linear_bf16(xb, bf16_weight(weight), _fp32_bias(bias), out, residual=res, nsplit=nsplit, epilogue=epilogue)
        ctx.save_for_backward(xb, weight, bias)
        ctx.cfg = (nsplit, epilogue, residual is not None)
        return out

    @staticmethod
    def backward(ctx, g):
        xb, weight, bias = ctx.saved_tensors
        nsplit, epilogue, has_res = ctx.cfg
        wb = bf16_weight(weight)
        if nsplit > 1:
            return LinearFn._backward_split(xb, weight, bias, wb, g.contiguous())
        g = g.contiguous()
        g_res = g if has_res else None
        if epilogue == pshattn.EPI_SWIGLU:
            # the pre-activation [gate | up] is recomputed on the native GEMM, its gradient by one fused kernel
            y = torch.empty(xb.shape[0], wb.shape[0], dtype=torch.bfloat16, device=xb.device)
            pshattn.linear_bf16(xb, wb, _fp32_bias(bias), y)
            gy = torch.empty_like(y)
            pshattn.swiglu_bwd_bf16(y, g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16), gy)
            g = gy
        elif epilogue == pshattn.EPI_GELU:
            # the same for the tanh-form GELU epilogue
            y = torch.empty(xb.shape[0], wb.shape[0], dtype=torch.bfloat16, device=xb.device)
            pshattn.linear_bf16(xb, wb, _fp32_bias(bias), y)
            gy = torch.empty_like(y)
            pshattn.gelu_bwd_bf16(y, g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16), gy, tanh_form=True)
            g = gy
        # gx = g W: the native GEMM computes A B^T, so W^T ([in, out], a small matrix) is materialised
        gx = torch.empty(g.shape[0], wb.shape[1], dtype=torch.bfloat16, device=g.device)
        pshattn.linear_bf16(g, wb.t().contiguous(), None, gx)
        gw, gb = _param_grads(g, xb, weight, bias)
        return gx, gw, gb, g_res, None, None


def _split_backward(xb, weight, bias, wb, g):
    """Backward of a projection whose output is nsplit separate matrices: g is the packed gradient [S, M, C]."""
    s, m, c = g.shape
    # grad_x = sum_s g[s] W_s as one GEMM over the slices; W_s^T ([in, C] per slice) is a small matrix
    wt = wb.view(s, c, wb.shape[1]).transpose(1, 2).contiguous()
    gx = torch.empty(m, wb.shape[1], dtype=torch.bfloat16, device=g.device)
    pshattn.linear_ksplit_bf16(g, wt, gx)
    parts = [_param_grads(g[i], xb, weight, bias[i * c:(i + 1) * c] if bias is not None else None) for i in range(s)]
    gw = torch.cat([p[0] for p in parts], dim=0)
    gb = torch.cat([p[1] for p in parts], dim=0) if bias is not None else None
    return gx, gw, gb, None, None, None


LinearFn._backward_split = staticmethod(_split_backward)


def linear(x, weight, bias=None, residual=None, nsplit=1, epilogue=pshattn.EPI_NONE):
    if not torch.is_grad_enabled() and x.dtype == torch.bfloat16 and x.is_contiguous():
        # inference: the same GEMM without the autograd bookkeeping of a Function call
        return linear_inference(x, weight, bias, None if residual is None else residual.contiguous(), nsplit, epilogue)
    return LinearFn.apply(x, weight, bias, residual, nsplit, epilogue)


class LayerNormFn(Function):
    """LayerNorm (+ optional GELU) on the native kernels, forward and backward; with the fused GELU the backward
    recomputes the normalised rows, takes the gradient through the activation and runs the same native backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, gelu):
        xb = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        out = torch.empty_like(xb)
        pshattn.layernorm_bf16(xb, weight.detach().float().contiguous(), bias.detach().float().contiguous(), out, eps, gelu)
        ctx.save_for_backward(xb, weight, bias)
        ctx.cfg = (eps, gelu)
        return out

    @staticmethod
    def backward(ctx, g):
        xb, weight, bias = ctx.saved_tensors
        eps, gelu = ctx.cfg
        if xb.shape[1] <= 1024:
            gb16 = (g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)).contiguous()
            if gelu:
                y = torch.empty_like(xb)
                pshattn.layernorm_bf16(xb, weight.detach().float().contiguous(), bias.detach().float().contiguous(), y, eps, False)
                gy = torch.empty_like(y)
                pshattn.gelu_bwd_bf16(y, gb16, gy, tanh_form=False)
                gb16 = gy
            gx = torch.empty_like(xb)
            gw = torch.empty(xb.shape[1], dtype=torch.float32, device=xb.device)
            gb = torch.empty_like(gw)
            pshattn.layernorm_bwd_bf16(xb, gb16, weight.detach().float().contiguous(), gx, gw, gb, eps)
            return gx, gw.to(weight.dtype), gb.to(bias.dtype), None, None
        with torch.enable_grad():
            xf = xb.float().requires_grad_(True)
            wf = weight.detach().float().requires_grad_(True)
            bf = bias.detach().float().requires_grad_(True)
            y = torch.nn.functional.layer_norm(xf, (xf.shape[-1],), wf, bf, eps)
            if gelu:
                y = torch.nn.functional.gelu(y)
            gx, gw, gb = torch.autograd.grad(y, (xf, wf, bf), g.float())
        return gx.to(xb.dtype), gw.to(weight.dtype), gb.to(bias.dtype), None, None


def layer_norm(x, weight, bias, eps=1e-5, gelu=False):
    if not torch.is_grad_enabled() and x.dtype == torch.bfloat16 and x.is_contiguous():
        out = torch.empty_like(x)
        pshattn.layernorm_bf16(x, _fp32_param(weight), _fp32_param(bias), out, eps, gelu)
        return out
    return LayerNormFn.apply(x, weight, bias, eps, gelu)


def apply_norm(norm: torch.nn.Module, x: torch.Tensor, act: torch.nn.Module = None):
    """Run a user-supplied normalisation (and activation) module.  nn.LayerNorm over the channel dimension goes to
    the native kernel, with an nn.GELU activation fused; anything else (BatchNorm, custom modules) runs as given,
    in the dtype of its parameters."""
    if (isinstance(norm, torch.nn.LayerNorm) and x.is_cuda and x.dim() == 2 and norm.elementwise_affine
            and norm.bias is not None and tuple(norm.normalized_shape) == (x.shape[-1],) and x.shape[-1] % 8 == 0):
        fuse = isinstance(act, torch.nn.GELU) and getattr(act, "approximate", "none") == "none"
        y = layer_norm(x, norm.weight, norm.bias, norm.eps, gelu=fuse)
        return y if (act is None or fuse) else act(y)
    if norm is not None:
        p = next(norm.parameters(), None)
        y = norm(x.to(p.dtype) if p is not None and p.dtype != x.dtype else x)
    else:
        y = x
    y = act(y) if act is not None else y
    return y.to(torch.bfloat16) if y.dtype != torch.bfloat16 else y
