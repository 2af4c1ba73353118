"""GPU parity of the native LayerNorm forward and backward against fp32 torch (the reference takes both from
TransformerEngine / nn.LayerNorm, flash3dxfmr/layers/stage.py:67,95).  Forward and dx are bf16 outputs: they may
differ from the fp32 result by the final rounding (2^-8 relative) plus fp32 reassociation; the parameter gradients
are fp32 sums over all rows and are compared relative to their magnitude."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(dev, rows, c, seed):
    g = torch.Generator(dev).manual_seed(seed)
    x = (torch.randn(rows, c, device=dev, generator=g) * 1.5 + 0.3).bfloat16()
    w = torch.randn(c, device=dev, generator=g) * 0.5 + 1.0
    b = torch.randn(c, device=dev, generator=g) * 0.2
    go = torch.randn(rows, c, device=dev, generator=g).bfloat16()
    return x, w, b, go


@pytest.mark.parametrize("rows,c", [(1, 32), (1000, 32), (4097, 64), (777, 128), (2048, 256), (513, 512), (300, 1024), (65, 24)])
@pytest.mark.parametrize("gelu", [False, True])
def test_layernorm_forward(cuda_device, rows, c, gelu):
    from flash3dtransformer_b200.lib import pshattn
    x, w, b, _ = _inputs(cuda_device, rows, c, rows + c)
    out = torch.full_like(x, float("nan"))
    pshattn.layernorm_bf16(x, w, b, out, 1e-5, gelu)
    ref = torch.nn.functional.layer_norm(x.float(), (c,), w, b, 1e-5)
    if gelu:
        ref = torch.nn.functional.gelu(ref)
    assert torch.isfinite(out.float()).all()
    assert ((out.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 2e-3).all()


@pytest.mark.parametrize("rows,c", [(1, 32), (1000, 32), (70001, 64), (777, 128), (20000, 256), (513, 512), (300, 1024), (65, 24)])
def test_layernorm_backward(cuda_device, rows, c):
    from flash3dtransformer_b200.lib import pshattn
    x, w, b, go = _inputs(cuda_device, rows, c, 3 * rows + c)
    dx = torch.full_like(x, float("nan"))
    dw = torch.full((c,), float("nan"), device=cuda_device)
    db = torch.full((c,), float("nan"), device=cuda_device)
    pshattn.layernorm_bwd_bf16(x, go, w, dx, dw, db, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.clone().requires_grad_(True)
    bf = b.clone().requires_grad_(True)
    y = torch.nn.functional.layer_norm(xf, (c,), wf, bf, 1e-5)
    rx, rw, rb = torch.autograd.grad(y, (xf, wf, bf), go.float())
    assert torch.isfinite(dx.float()).all() and torch.isfinite(dw).all() and torch.isfinite(db).all()
    assert ((dx.float() - rx).abs() <= rx.abs() * 2.0 ** -7 + 3e-3).all()
    scale_w = rw.abs().max().item() + 1e-3
    assert (dw - rw).abs().max().item() <= 1e-4 * scale_w + 1e-4 * rows ** 0.5
    assert (db - rb).abs().max().item() <= 1e-4 * (rb.abs().max().item() + 1e-3) + 1e-4 * rows ** 0.5
    # same bits on a second run (fixed summation order)
    dw2, db2 = torch.empty_like(dw), torch.empty_like(db)
    pshattn.layernorm_bwd_bf16(x, go, w, torch.empty_like(dx), dw2, db2, 1e-5)
    assert torch.equal(dw, dw2) and torch.equal(db, db2)


def test_layernorm_autograd_path(cuda_device):
    from flash3dtransformer_b200.layers.functional import layer_norm
    x, w, b, go = _inputs(cuda_device, 3000, 128, 9)
    xr = x.clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    y = layer_norm(xr, wr, br)
    y.backward(go)
    xf = x.float().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xf, (128,), w, b, 1e-5)
    rx, = torch.autograd.grad(ref, xf, go.float())
    assert ((xr.grad.float() - rx).abs() <= rx.abs() * 2.0 ** -7 + 3e-3).all()
    assert wr.grad is not None and br.grad is not None


def test_layernorm_gelu_autograd_path(cuda_device):
    """LayerNorm with the fused GELU: the backward recomputes the normalised rows (bf16), takes the gradient through
    the activation and runs the native LayerNorm backward; compared with fp32 autograd of the same formula.  The extra
    bf16 rounding of the recomputed rows allows 2^-6 relative."""
    from flash3dtransformer_b200.layers.functional import layer_norm
    x, w, b, go = _inputs(cuda_device, 5000, 64, 4)
    xr = x.clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    y = layer_norm(xr, wr, br, gelu=True)
    y.backward(go)
    xf = x.float().requires_grad_(True)
    wf, bf = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = torch.nn.functional.gelu(torch.nn.functional.layer_norm(xf, (64,), wf, bf, 1e-5))
    rx, rw, rb = torch.autograd.grad(ref, (xf, wf, bf), go.float())
    err = (xr.grad.float() - rx).abs()
    assert (err <= rx.abs() * 2.0 ** -6 + 2e-2).all(), err.max().item()
    assert err.mean().item() <= 2e-3 * rx.abs().mean().item() + 1e-4
    assert (wr.grad - rw).abs().max().item() <= 5e-3 * rw.abs().max().item() + 5e-2
    assert (br.grad - rb).abs().max().item() <= 5e-3 * rb.abs().max().item() + 5e-2
