"""Whole-model tests: the Flash3D module tree runs forward (and backward) on the native kernels, as in the
reference's integration smoke test (tests/test_psh_hourglass.py:51-163), plus a forward check against a plain
torch restatement of one transformer block."""
import numpy as np
import pytest
import torch

from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu


def _batch(dev, sizes, seed=0):
    c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=seed)
    return (torch.from_numpy(c32.astype(np.float16)).to(dev), torch.from_numpy(seps.astype(np.uint32)).to(dev))


def test_two_level_backbone_forward(cuda_device):
    from flash3dtransformer_b200 import configs
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(0)
    model = configs.flash3d_backbone(channels=(32, 64), depths=(2, 2)).to(cuda_device)
    coords, seps = _batch(cuda_device, [30000, 22000, 41000])
    with torch.no_grad():
        out = model(coords, coords, seps)
    pshattn.device_status()
    assert out.shape == (-(-coords.shape[0] // (512 * 8 * 6)) * 512 * 8 * 6, 32)
    assert out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    with torch.no_grad():
        again = model(coords, coords, seps)
    assert torch.equal(out, again)            # the whole forward is deterministic


def test_xfmr_block_matches_torch(cuda_device):
    """One XFMR block against fp32 torch: LayerNorm, QKV, per-scope softmax attention, projection + residual,
    LayerNorm, SwiGLU MLP + residual."""
    from flash3dtransformer_b200 import layers
    from flash3dtransformer_b200.psh import bucket_scope
    torch.manual_seed(1)
    c, heads, bucket, k = 64, 2, 256, 2
    n = bucket * k * 3
    blk = layers.XFMR(c, 4 * c, heads, bucket, True, bucket_scope.SwinPlan("swin", bucket, k, 0), torch.nn.LayerNorm).to(cuda_device)
    x = torch.randn(n, c, device=cuda_device).bfloat16()
    with torch.no_grad():
        out = blk(None, x, None).float()
        xf = x.float()
        h = torch.nn.functional.layer_norm(xf, (c,), blk.norm.weight, blk.norm.bias)
        qkv = h @ blk.bwa.qkv.weight.t() + blk.bwa.qkv.bias
        q, kk, v = (t.view(n // (bucket * k), bucket * k, heads, c // heads).transpose(1, 2) for t in qkv.chunk(3, -1))
        a = torch.nn.functional.scaled_dot_product_attention(q, kk, v).transpose(1, 2).reshape(n, c)
        mid = a @ blk.bwa.proj.weight.t() + blk.bwa.proj.bias + xf
        m = blk.mlp.mlp
        h2 = torch.nn.functional.layer_norm(mid, (c,), m.layer_norm_weight, m.layer_norm_bias)
        y = h2 @ m.fc1_weight.t() + m.fc1_bias
        f = y.shape[1] // 2
        ref = (torch.nn.functional.silu(y[:, :f]) * y[:, f:]) @ m.fc2_weight.t() + m.fc2_bias + mid
    err = (out - ref).abs()
    assert err.max().item() <= 6e-2 and (err.mean() / ref.abs().mean()).item() <= 8e-3


def test_backbone_forward_matches_cpu_oracle(cuda_device):
    """Three-level backbone on two small scans against the composed CPU oracle (fp32 with bf16 storage rounding).
    Every layer re-rounds to bf16, so the tolerance is the per-layer bar accumulated over ~10 layers."""
    from flash3dtransformer_b200 import configs
    from oracle import backbone_oracle
    torch.manual_seed(0)
    model = configs.flash3d_backbone(channels=(32, 64, 128), depths=(1, 1, 1), bucket_size=256, scope_size=2)
    c32, seps = synthetic.batch(synthetic.lidar_scan, [5000, 3500], seed=2)
    c16 = c32.astype(np.float16)
    ref = backbone_oracle.flash3d_forward(model, c16, seps)
    model = model.to(cuda_device)
    with torch.no_grad():
        out = model(torch.from_numpy(c16).to(cuda_device), None, torch.from_numpy(seps.astype(np.uint32)).to(cuda_device))
    out = out.float().cpu()
    assert out.shape == ref.shape
    err = (out - ref).abs()
    scaled = err / ref.abs().clamp(min=1.0)       # coordinates in metres make some features large: 1 bf16 ulp at 64 is 0.25
    assert scaled.max().item() <= 0.1, scaled.max().item()
    assert (err.mean() / ref.abs().mean()).item() <= 1e-2, (err.mean() / ref.abs().mean()).item()
    # rows behind the last scene (tail padding) carry no garbage
    assert torch.isfinite(out).all()


def test_backbone_forward_backward_runs(cuda_device):
    """The reference's integration smoke test (tests/test_psh_hourglass.py:51-163): a two-level model runs forward
    and backward, and gradients reach every parameter."""
    from flash3dtransformer_b200 import configs
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(0)
    model = configs.flash3d_backbone(channels=(32, 64), depths=(2, 2)).to(cuda_device)
    coords, seps = _batch(cuda_device, [30000, 22000])
    out = model(coords, coords, seps)
    loss = out.float().mean()
    loss.backward()
    pshattn.device_status()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert not missing, missing
    for n, p in model.named_parameters():
        assert torch.isfinite(p.grad).all(), n
    assert model.psh_scatter.lin.weight.grad.abs().sum().item() > 0          # tests/test_psh.py:367-396


def test_xfmr_block_gradients_match_torch(cuda_device):
    """Gradients of one XFMR block (attention backward kernel + torch GEMM backward) against autograd of an fp32
    torch restatement of the block."""
    from flash3dtransformer_b200 import layers
    from flash3dtransformer_b200.psh import bucket_scope
    torch.manual_seed(3)
    c, heads, bucket, k = 64, 2, 256, 2
    n = bucket * k * 2
    blk = layers.XFMR(c, 4 * c, heads, bucket, True, bucket_scope.SwinPlan("swin", bucket, k, 0), torch.nn.LayerNorm).to(cuda_device)
    x = torch.randn(n, c, device=cuda_device).bfloat16().requires_grad_(True)
    g = torch.randn(n, c, device=cuda_device).bfloat16()
    blk(None, x, None).backward(g)
    got_x = x.grad.float()
    got_w = blk.bwa.qkv.weight.grad.float().clone()
    blk.zero_grad()
    xf = x.detach().float().requires_grad_(True)
    h = torch.nn.functional.layer_norm(xf, (c,), blk.norm.weight, blk.norm.bias)
    qkv = h @ blk.bwa.qkv.weight.t() + blk.bwa.qkv.bias
    q, kk, v = (t.view(n // (bucket * k), bucket * k, heads, c // heads).transpose(1, 2) for t in qkv.chunk(3, -1))
    a = torch.nn.functional.scaled_dot_product_attention(q, kk, v).transpose(1, 2).reshape(n, c)
    mid = a @ blk.bwa.proj.weight.t() + blk.bwa.proj.bias + xf
    m = blk.mlp.mlp
    h2 = torch.nn.functional.layer_norm(mid, (c,), m.layer_norm_weight, m.layer_norm_bias)
    y = h2 @ m.fc1_weight.t() + m.fc1_bias
    f = y.shape[1] // 2
    out = (torch.nn.functional.silu(y[:, :f]) * y[:, f:]) @ m.fc2_weight.t() + m.fc2_bias + mid
    out.backward(g.float())
    for name, got, ref in (("x", got_x, xf.grad), ("qkv.weight", got_w, blk.bwa.qkv.weight.grad.float())):
        err = (got - ref).abs()
        assert err.max().item() <= 0.05 * ref.abs().max().item() + 1e-3, (name, err.max().item(), ref.abs().max().item())
        assert (err.mean() / ref.abs().mean()).item() <= 2e-2, (name, (err.mean() / ref.abs().mean()).item())


def test_input_features_and_input_order(cuda_device):
    """The two switches beyond the reference: input features scattered into bucket order and the result gathered
    back to the order of the input points, forward and backward."""
    from flash3dtransformer_b200 import configs
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(0)
    base = configs.flash3d_backbone(channels=(32, 64), depths=(2, 2)).to(cuda_device)
    full = configs.flash3d_backbone(channels=(32, 64), depths=(2, 2), scatter_input_feat=True,
                                    restore_input_order=True).to(cuda_device)
    full.load_state_dict(base.state_dict())
    coords, seps = _batch(cuda_device, [30000, 22000])
    n = coords.shape[0]
    zeros = torch.zeros(n, 32, dtype=torch.bfloat16, device=cuda_device, requires_grad=True)
    ref = base(coords, coords, seps)                                   # bucket order, [pad_to, 32]
    out = full(coords, zeros, seps)                                    # input order, [n, 32]
    assert out.shape == (n, 32)
    # with zero features the result is the reference-order result, permuted: check through the coordinates' own scatter
    from flash3dtransformer_b200.psh import psh_main as pm
    pad_to = ref.shape[0]
    _, buffers = pm.batch_bucket_scatter(coords, seps, 512, pad_to, 2)
    out2in, in2out = pm.scatter_index(buffers, seps, pad_to)
    assert torch.equal(out, ref[in2out.long()])
    # gradients: d(sum of out * w)/d(input_feat) arrives in input order and is finite; rows are not mixed up
    w = torch.randn(n, 32, device=cuda_device)
    (out.float() * w).sum().backward()
    pshattn.device_status()
    assert zeros.grad is not None and zeros.grad.shape == (n, 32) and torch.isfinite(zeros.grad.float()).all()
    assert zeros.grad.abs().sum().item() > 0
    # non-zero features change the result
    feat = torch.randn(n, 32, device=cuda_device).to(torch.bfloat16)
    with torch.no_grad():
        out2 = full(coords, feat, seps)
    assert not torch.equal(out2, out)


def test_batchnorm_pool_wrappers_forward_backward(cuda_device):
    """The reference's whole-model test wraps pooling and unpooling in BatchNorm1d + GELU
    (tests/test_psh_hourglass.py:103-106): user-supplied normalisation modules run as given next to the native
    kernels, forward and backward."""
    import dataclasses
    from torch import nn
    from flash3dtransformer_b200 import configs, layers
    from flash3dtransformer_b200.lib import pshattn
    torch.manual_seed(0)
    specs = configs.hourglass_specs((32, 64), (2, 2))
    specs = [dataclasses.replace(s, pool_norm=nn.BatchNorm1d, unpool_norm=nn.BatchNorm1d) for s in specs]
    model = layers.Flash3D(specs, 512, 8, 2).to(cuda_device).train()
    coords, seps = _batch(cuda_device, [20000, 26000], seed=4)
    out = model(coords, coords, seps)
    assert out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    out.float().square().mean().backward()
    pshattn.device_status()
    for n, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), n
    assert any(isinstance(m, nn.BatchNorm1d) for m in model.modules())


def test_inference_reuses_level_buffers(cuda_device):
    """Without autograd the intermediate buffers of every level are planned once per batch signature: the second
    forward pass over a batch of the same scene sizes allocates only its activations (peak memory does not grow, the
    PSH / sub-bucket tables are the same objects) and gives the same bits; another signature gets its own plan; with
    autograd nothing is shared."""
    from flash3dtransformer_b200 import configs
    from flash3dtransformer_b200.psh import plan, psh_main
    torch.manual_seed(0)
    model = configs.flash3d_backbone(channels=(32, 64), depths=(1, 1)).to(cuda_device)
    coords, seps = _batch(cuda_device, [30000, 22000], seed=1)
    coords2, seps2 = _batch(cuda_device, [30000, 22000], seed=2)
    plan.clear()
    with torch.no_grad():
        a1 = model(coords, None, seps)
        n_plans = len(plan._pool)
        assert n_plans >= 3                                   # PSH tables, one sub-bucket plan, log-sum-exp rows
        b1 = model(coords2, None, seps2)                      # same signature, other points: the plans are reused
        assert len(plan._pool) == n_plans
        a2 = model(coords, None, seps)
        assert torch.equal(a1, a2) and not torch.equal(a1, b1)
        other, oseps = _batch(cuda_device, [25000, 26000], seed=3)
        model(other, None, oseps)
        assert len(plan._pool) > n_plans
    with plan.level_buffers():
        x = psh_main.BucketScatterBuffers.create_buffers(coords, seps, 512, coords.shape[0], 64)
        y = psh_main.BucketScatterBuffers.create_buffers(coords, seps, 512, coords.shape[0], 64)
        assert x is y
    x = psh_main.BucketScatterBuffers.create_buffers(coords, seps, 512, coords.shape[0], 64)
    y = psh_main.BucketScatterBuffers.create_buffers(coords, seps, 512, coords.shape[0], 64)
    assert x is not y and x.bucket_id.data_ptr() != y.bucket_id.data_ptr()
    n_before = len(plan._pool)
    out = model(coords, None, seps)                           # autograd on: private buffers
    assert len(plan._pool) == n_before and out.requires_grad
    plan.clear()
