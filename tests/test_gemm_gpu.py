"""GPU parity of the tcgen05 GEMM against an fp32 torch reference.  Tolerance (bf16 outputs of unit scale):
max abs <= 2e-2 against the fp32 reference, and mean|err| / mean|ref| exceeds the floor set by rounding the exact
result to bf16 (about 1.4e-3 mean relative) by at most 1e-3."""
import pytest
import torch

from conftest import record_parity

pytestmark = pytest.mark.gpu


def _check(out, ref, max_abs=2e-2, mean_rel=1e-3):
    err = (out.float() - ref).abs()
    assert torch.isfinite(out.float()).all()
    scaled = err / ref.abs().clamp(min=1.0)          # absolute below 1, relative above (bf16 keeps 8 bits)
    rel = (err.mean() / ref.abs().mean()).item()
    floor = ((ref.to(out.dtype).float() - ref).abs().mean() / ref.abs().mean()).item()
    record_parity("gemm", max_abs_raw=err.max().item(), max_abs_scaled=scaled.max().item(), mean_rel_raw=rel,
                  rounding_floor=floor, ref_abs_max=ref.abs().max().item(), bound_max_abs=max_abs, bound_mean_rel_excess=mean_rel)
    assert scaled.max().item() <= max_abs, f"max abs {scaled.max().item()}"
    assert rel <= floor + mean_rel, f"mean rel {rel} (bf16 rounding floor {floor})"


def _mk(dev, m, n, k, seed=0):
    g = torch.Generator(dev).manual_seed(seed)
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w = (torch.randn(n, k, device=dev, generator=g) / k ** 0.5).bfloat16()
    b = torch.randn(n, device=dev, generator=g) * 0.1
    return x, w, b


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 256), (1000, 96, 32), (4096, 768, 256), (333, 512, 512),
                                   (2048, 64, 128), (777, 1536, 512), (128, 32, 2048), (5000, 256, 40)])
def test_linear_plain(cuda_device, m, n, k):
    from flash3dtransformer_b200.lib import pshattn
    x, w, b = _mk(cuda_device, m, n, k)
    out = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_bf16(x, w, b, out)
    pshattn.device_status()
    _check(out, x.float() @ w.float().t() + b)
    out2 = torch.empty_like(out)
    pshattn.linear_bf16(x, w, None, out2)
    _check(out2, x.float() @ w.float().t())


@pytest.mark.parametrize("m,c", [(1024, 32), (3000, 64), (2048, 128), (1536, 256), (640, 512)])
def test_qkv_split_and_residual(cuda_device, m, c):
    from flash3dtransformer_b200.lib import pshattn
    x, w, b = _mk(cuda_device, m, 3 * c, c, seed=1)
    qkv = torch.full((3, m, c), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_bf16(x, w, b, qkv, nsplit=3)
    ref = x.float() @ w.float().t() + b
    for i in range(3):
        _check(qkv[i], ref[:, i * c:(i + 1) * c])
    xw, ww, bw = _mk(cuda_device, m, c, c, seed=2)
    out = torch.empty(m, c, device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_bf16(xw, ww, bw, out, residual=x)
    pshattn.device_status()
    _check(out, xw.float() @ ww.float().t() + bw + x.float(), max_abs=4e-2)


# (1000, 32, 128) and (3001, 64, 128): one column tile, where the bias rides in the product
@pytest.mark.parametrize("m,c,f", [(1024, 128, 256), (700, 64, 256), (2048, 256, 1024), (1000, 32, 128), (3001, 64, 128), (513, 32, 64)])
def test_swiglu_and_gelu(cuda_device, m, c, f):
    from flash3dtransformer_b200.lib import pshattn
    x, w, b = _mk(cuda_device, m, 2 * f, c, seed=3)
    out = torch.empty(m, f, device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_bf16(x, w, b, out, epilogue=pshattn.EPI_SWIGLU)
    y = x.float() @ w.float().t() + b
    _check(out, torch.nn.functional.silu(y[:, :f]) * y[:, f:])
    out2 = torch.empty(m, 2 * f, device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_bf16(x, w, b, out2, epilogue=pshattn.EPI_GELU)
    pshattn.device_status()
    _check(out2, torch.nn.functional.gelu(y, approximate="tanh"))


def test_gemm_sm_bf16_export(cuda_device):
    """The reference's own GEMM test: 128x256 @ 256x128, atol = rtol = 1e-2 (tests/test_gemm.py:26-43)."""
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(2)
    a = torch.randn(128, 256, device=cuda_device).bfloat16() / 16
    b = torch.randn(256, 128, device=cuda_device).bfloat16() / 16
    o = torch.zeros(128, 128, device=cuda_device, dtype=torch.bfloat16)
    pshattn.gemm_sm_bf16(a, b, o)
    assert torch.allclose(o.float(), (a.float() @ b.float()), atol=1e-2, rtol=1e-2)
    a = torch.randn(300, 72, device=cuda_device).bfloat16() / 8
    b = torch.randn(72, 40, device=cuda_device).bfloat16() / 8
    o = torch.zeros(300, 40, device=cuda_device, dtype=torch.bfloat16)
    pshattn.gemm_sm_bf16(a, b, o)
    assert torch.allclose(o.float(), (a.float() @ b.float()), atol=1e-2, rtol=1e-2)


def test_gemm_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    x = torch.zeros(16, 12, device=cuda_device, dtype=torch.bfloat16)
    w = torch.zeros(8, 12, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="multiples of 8"):
        pshattn.linear_bf16(x, w, None, torch.zeros(16, 8, device=cuda_device, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="dtype"):
        pshattn.linear_bf16(x.float(), w, None, torch.zeros(16, 8, device=cuda_device, dtype=torch.bfloat16))


@pytest.mark.parametrize("rows,c", [(1, 32), (1000, 32), (70001, 64), (4096, 512), (513, 2048)])
def test_coord_embed(cuda_device, rows, c):
    """The 3 -> C coordinate embedding (te.Linear(3, emb_dim) in the reference, flash3dxfmr/layers/psh_ops.py:62)
    against an fp32 torch reference; the result differs from it only by the final rounding to bf16."""
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(rows + c)
    x = (torch.randn(rows, 3, device=cuda_device, generator=g) * 20).half()
    w = torch.randn(c, 3, device=cuda_device, generator=g) * 0.5
    b = torch.randn(c, device=cuda_device, generator=g)
    out = torch.full((rows, c), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    pshattn.coord_embed_bf16(x, w, b, out)
    ref = x.float() @ w.t() + b
    assert torch.isfinite(out.float()).all()
    # one bf16 rounding of a value computed in fp32 (the FMA order may differ from torch's by an ulp of fp32)
    assert ((out.float() - ref).abs() <= ref.abs() * 2.0 ** -8 + 1e-6).all()


def test_linear_input_gradient_runs_native(cuda_device):
    """The autograd backward of the projection computes g W on the native GEMM; compare with fp32 autograd."""
    from flash3dtransformer_b200.layers.functional import LinearFn
    g = torch.Generator(cuda_device).manual_seed(5)
    x = torch.randn(1024, 64, device=cuda_device, generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(96, 64, device=cuda_device, generator=g) / 8).requires_grad_(True)
    b = torch.zeros(96, device=cuda_device, requires_grad=True)
    y = LinearFn.apply(x, w, b, None, 1, 0)
    gy = torch.randn(1024, 96, device=cuda_device, generator=g).bfloat16()
    y.backward(gy)
    ref_gx = gy.float() @ w.detach().bfloat16().float()
    _check(x.grad, ref_gx)
    ref_gw = gy.float().t() @ x.detach().float()
    assert (w.grad - ref_gw).abs().max().item() <= 2e-2 * ref_gw.abs().max().item() + 1e-2


@pytest.mark.parametrize("rows,f", [(1, 8), (1000, 128), (4097, 256), (333, 2048)])
def test_swiglu_backward(cuda_device, rows, f):
    """Gradient of silu(gate) * up with respect to [gate | up] against fp32 autograd (bf16 outputs)."""
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(rows + f)
    y = (torch.randn(rows, 2 * f, device=cuda_device, generator=g) * 2).bfloat16()
    go = torch.randn(rows, f, device=cuda_device, generator=g).bfloat16()
    out = torch.full_like(y, float("nan"))
    pshattn.swiglu_bwd_bf16(y, go, out)
    yf = y.float().requires_grad_(True)
    z = torch.nn.functional.silu(yf[:, :f]) * yf[:, f:]
    ref, = torch.autograd.grad(z, yf, go.float())
    assert torch.isfinite(out.float()).all()
    assert ((out.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-3).all()


@pytest.mark.parametrize("rows,c,tanh_form", [(1, 8, False), (1000, 128, False), (4097, 256, True), (333, 2048, True), (70001, 32, False)])
def test_gelu_backward(cuda_device, rows, c, tanh_form):
    """Gradient of gelu(y) (exact and tanh form) against fp32 autograd; the output is one bf16 rounding away."""
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(rows + c)
    y = (torch.randn(rows, c, device=cuda_device, generator=g) * 2).bfloat16()
    go = torch.randn(rows, c, device=cuda_device, generator=g).bfloat16()
    out = torch.full_like(y, float("nan"))
    pshattn.gelu_bwd_bf16(y, go, out, tanh_form=tanh_form)
    yf = y.float().requires_grad_(True)
    z = torch.nn.functional.gelu(yf, approximate="tanh" if tanh_form else "none")
    ref, = torch.autograd.grad(z, yf, go.float())
    assert torch.isfinite(out.float()).all()
    assert ((out.float() - ref).abs() <= ref.abs() * 2.0 ** -7 + 1e-3).all()


@pytest.mark.parametrize("rows,c", [(1, 32), (1000, 32), (70001, 64), (4096, 512), (513, 2048), (300000, 32)])
def test_coord_embed_backward(cuda_device, rows, c):
    """Parameter gradients of the 3 -> C embedding against float64 sums; same bits on a second run; and through autograd
    of the layer function."""
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.layers.functional import CoordEmbedFn
    g = torch.Generator(cuda_device).manual_seed(rows + c)
    x = (torch.randn(rows, 3, device=cuda_device, generator=g) * 20).half()
    go = torch.randn(rows, c, device=cuda_device, generator=g).bfloat16()
    gw = torch.full((c, 3), float("nan"), device=cuda_device)
    gb = torch.full((c,), float("nan"), device=cuda_device)
    pshattn.coord_embed_bwd(x, go, gw, gb)
    ref_w = go.double().t() @ x.double()
    ref_b = go.double().sum(0)
    scale_w = (go.float().abs().t() @ x.float().abs()).max().item()
    assert (gw.double() - ref_w).abs().max().item() <= 1e-5 * scale_w + 1e-6
    assert (gb.double() - ref_b).abs().max().item() <= 1e-5 * go.float().abs().sum(0).max().item() + 1e-6
    gw2, gb2 = torch.empty_like(gw), torch.empty_like(gb)
    pshattn.coord_embed_bwd(x, go, gw2, gb2)
    assert torch.equal(gw, gw2) and torch.equal(gb, gb2)
    w = (torch.randn(c, 3, device=cuda_device, generator=g) * 0.5).requires_grad_(True)
    b = torch.randn(c, device=cuda_device, generator=g).requires_grad_(True)
    CoordEmbedFn.apply(x, w, b).backward(go)
    assert torch.equal(w.grad, gw) and torch.equal(b.grad, gb)


def test_gelu_linear_gradients(cuda_device):
    """LinearFn with the GELU epilogue: input, weight and bias gradients against fp32 autograd."""
    from flash3dtransformer_b200.layers.functional import LinearFn
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(23)
    x = torch.randn(2048, 64, device=cuda_device, generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(128, 64, device=cuda_device, generator=g) / 8).requires_grad_(True)
    b = (torch.randn(128, device=cuda_device, generator=g) * 0.1).requires_grad_(True)
    y = LinearFn.apply(x, w, b, None, 1, pshattn.EPI_GELU)
    gy = torch.randn(2048, 128, device=cuda_device, generator=g).bfloat16()
    y.backward(gy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().bfloat16().float().requires_grad_(True)
    br = b.detach().clone().requires_grad_(True)
    torch.nn.functional.gelu(xr @ wr.t() + br, approximate="tanh").backward(gy.float())
    _check(x.grad, xr.grad)
    assert (w.grad - wr.grad).abs().max().item() <= 2e-2 * wr.grad.abs().max().item() + 1e-2
    assert (b.grad - br.grad).abs().max().item() <= 2e-2 * br.grad.abs().max().item() + 1e-2


@pytest.mark.parametrize("rows,c", [(1, 8), (1000, 96), (70001, 32), (5000, 2048), (63, 512), (3000, 4096), (777, 2056)])
def test_colsum(cuda_device, rows, c):
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(rows + c)
    x = torch.randn(rows, c, device=cuda_device, generator=g).bfloat16()
    out = torch.full((c,), float("nan"), device=cuda_device)
    pshattn.colsum_bf16(x, out)
    ref = x.double().sum(0)
    assert (out.double() - ref).abs().max().item() <= 1e-5 * x.float().abs().sum(0).max().item() + 1e-6
    out2 = torch.empty_like(out)
    pshattn.colsum_bf16(x, out2)
    assert torch.equal(out, out2)


def test_swiglu_linear_gradients(cuda_device):
    """LinearFn with the SwiGLU epilogue: input, weight and bias gradients against fp32 autograd."""
    from flash3dtransformer_b200.layers.functional import LinearFn
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(21)
    x = torch.randn(2048, 64, device=cuda_device, generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(256, 64, device=cuda_device, generator=g) / 8).requires_grad_(True)
    b = (torch.randn(256, device=cuda_device, generator=g) * 0.1).requires_grad_(True)
    y = LinearFn.apply(x, w, b, None, 1, pshattn.EPI_SWIGLU)
    gy = torch.randn(2048, 128, device=cuda_device, generator=g).bfloat16()
    y.backward(gy)
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().bfloat16().float().requires_grad_(True)
    bf = b.detach().clone().requires_grad_(True)
    pre = xf @ wf.t() + bf
    z = torch.nn.functional.silu(pre[:, :128]) * pre[:, 128:]
    rx, rw, rb = torch.autograd.grad(z, (xf, wf, bf), gy.float())
    # two bf16 roundings on the way (the pre-activation gradient, then the product with W)
    err = (x.grad.float() - rx).abs()
    assert err.max().item() <= 0.03 * rx.abs().max().item()
    assert (err.mean() / rx.abs().mean()).item() <= 8e-3
    assert (w.grad - rw).abs().max().item() <= 2e-2 * rw.abs().max().item() + 1e-2
    assert (b.grad - rb).abs().max().item() <= 2e-2 * rb.abs().max().item() + 1e-2


@pytest.mark.parametrize("s,m,n,k", [(3, 1024, 32, 32), (3, 3000, 64, 64), (3, 777, 128, 128), (3, 1536, 256, 256),
                                     (3, 640, 512, 512), (2, 333, 96, 40), (4, 129, 64, 200)])
def test_linear_ksplit(cuda_device, s, m, n, k):
    """Sum of slice products (one GEMM over the K slices): also a last row tile that runs into the next slice's rows
    and K that is not a multiple of the 64-column k-block."""
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(cuda_device).manual_seed(s * 1000 + m)
    x = torch.randn(s, m, k, device=cuda_device, generator=g).bfloat16()
    w = (torch.randn(s, n, k, device=cuda_device, generator=g) / (s * k) ** 0.5).bfloat16()
    out = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    pshattn.linear_ksplit_bf16(x, w, out)
    pshattn.device_status()
    ref = torch.einsum("smk,snk->mn", x.float(), w.float())
    _check(out, ref)
    b = torch.randn(n, device=cuda_device, generator=g) * 0.1
    res = torch.randn(m, n, device=cuda_device, generator=g).bfloat16()
    pshattn.linear_ksplit_bf16(x, w, out, bias=b, residual=res)
    _check(out, ref + b + res.float(), max_abs=4e-2)
    with pytest.raises(RuntimeError):
        pshattn.linear_ksplit_bf16(x, w[:, :, : k - 8].contiguous(), out)


def test_split_projection_gradients(cuda_device):
    """Backward of the Q/K/V projection (packed gradient [3, M, C]) against fp32 autograd."""
    from flash3dtransformer_b200.layers.functional import LinearFn
    g = torch.Generator(cuda_device).manual_seed(9)
    m, c = 2000, 64
    x = torch.randn(m, c, device=cuda_device, generator=g).bfloat16().requires_grad_(True)
    w = (torch.randn(3 * c, c, device=cuda_device, generator=g) / 8).requires_grad_(True)
    b = torch.zeros(3 * c, device=cuda_device, requires_grad=True)
    y = LinearFn.apply(x, w, b, None, 3, 0)                       # [3, m, c]
    gy = torch.randn(3, m, c, device=cuda_device, generator=g).bfloat16()
    y.backward(gy)
    flat = gy.permute(1, 0, 2).reshape(m, 3 * c).float()
    _check(x.grad, flat @ w.detach().bfloat16().float())
    ref_gw = flat.t() @ x.detach().float()
    assert (w.grad - ref_gw).abs().max().item() <= 2e-2 * ref_gw.abs().max().item() + 1e-2
    ref_gb = flat.sum(0)
    assert (b.grad - ref_gb).abs().max().item() <= 1e-3 * ref_gb.abs().max().item() + 1e-3


@pytest.mark.parametrize("m,n,k", [(1000, 32, 32), (4097, 96, 32), (3000, 256, 32), (5000, 64, 64), (2048, 192, 64),
                                   (1500, 128, 128), (777, 384, 128), (3001, 256, 256), (900, 512, 512), (640, 2048, 512),
                                   (1200, 64, 1024), (63, 40, 192), (1, 8, 64)])
def test_linear_wgrad(cuda_device, m, n, k):
    """grad_W = g^T x and grad_b = colsum(g) against fp32 torch; fp32 accumulation of exact bf16 products, so only the
    summation order differs: 1e-4 of the largest entry plus 1e-5 * sqrt(M)."""
    from flash3dtransformer_b200.lib import pshattn
    gen = torch.Generator(cuda_device).manual_seed(m + n + k)
    g = torch.randn(m, n, device=cuda_device, generator=gen).bfloat16()
    x = torch.randn(m, k, device=cuda_device, generator=gen).bfloat16()
    gw = torch.full((n, k), float("nan"), device=cuda_device)
    gb = torch.full((n,), float("nan"), device=cuda_device)
    pshattn.linear_wgrad_bf16(g, x, gw, gb)
    pshattn.device_status()
    ref_w = g.float().t() @ x.float()
    ref_b = g.float().sum(0)
    tol_w = 1e-4 * ref_w.abs().max().item() + 1e-5 * m ** 0.5
    assert torch.isfinite(gw).all() and (gw - ref_w).abs().max().item() <= tol_w, (gw - ref_w).abs().max().item()
    assert (gb - ref_b).abs().max().item() <= 1e-4 * ref_b.abs().max().item() + 1e-5 * m ** 0.5
    # without the bias gradient, and the same bits on a second run
    gw2 = torch.empty_like(gw)
    pshattn.linear_wgrad_bf16(g, x, gw2)
    assert torch.equal(gw, gw2)


def test_linear_wgrad_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    g = torch.zeros(16, 32, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        pshattn.linear_wgrad_bf16(g, torch.zeros(16, 48, device=cuda_device, dtype=torch.bfloat16), torch.zeros(32, 48, device=cuda_device))
    with pytest.raises(RuntimeError):
        pshattn.linear_wgrad_bf16(g, torch.zeros(15, 64, device=cuda_device, dtype=torch.bfloat16), torch.zeros(32, 64, device=cuda_device))
    assert pshattn.wgrad_supported(96, 32) and not pshattn.wgrad_supported(96, 48) and not pshattn.wgrad_supported(20, 64)
