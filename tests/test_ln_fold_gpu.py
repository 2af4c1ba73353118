"""LayerNorm folded into the projection GEMM (f3d_linear_fused) against the unfused pair (LayerNorm kernel, then GEMM)
and against fp32 torch; row sums written by a GEMM epilogue against the row-statistics kernel and torch; a transformer
block and a two-level backbone on the folded path against the unfused path."""
import numpy as np
import pytest
import torch

from conftest import record_parity
from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu


def _check(out, ref, name, max_abs=2e-2, mean_rel=1e-3):
    err = (out.float() - ref).abs()
    scaled = (err / ref.abs().clamp(min=1.0)).max().item()
    rel = (err.mean() / ref.abs().mean()).item()
    floor = ((ref.bfloat16().float() - ref).abs().mean() / ref.abs().mean()).item()
    record_parity(name, max_abs_raw=err.max().item(), max_abs_scaled=scaled, mean_rel_raw=rel, rounding_floor=floor,
                  ref_abs_max=ref.abs().max().item(), bound_max_abs=max_abs, bound_mean_rel_excess=mean_rel)
    assert torch.isfinite(out.float()).all()
    assert scaled <= max_abs, f"{name}: max abs {scaled}"
    assert rel <= floor + mean_rel, f"{name}: mean rel {rel} (floor {floor})"


@pytest.mark.parametrize("m,c,n,nsplit,epi", [(3000, 32, 96, 3, 0), (2048, 64, 192, 3, 0), (1500, 128, 1024, 1, 2),
                                              (1024, 256, 2048, 1, 2), (640, 512, 1536, 3, 0), (4096, 32, 256, 1, 2),
                                              (777, 128, 128, 1, 0)])
def test_folded_layernorm_matches_unfused_and_fp32(cuda_device, m, c, n, nsplit, epi):
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.layers import functional as F3
    dev = cuda_device
    g = torch.Generator(dev).manual_seed(m + c)
    # rows with a mean well away from zero and different scales, as residual streams have
    x = (torch.randn(m, c, device=dev, generator=g) * (0.5 + torch.rand(m, 1, device=dev, generator=g) * 3) +
         torch.randn(m, 1, device=dev, generator=g) * 2).bfloat16()
    # weights that bf16 holds exactly, as in the other GEMM tests: what is compared is the arithmetic, and the two
    # paths then differ in one rounding each (the fold rounds W * gamma, the unfused pair rounds the normalised rows)
    w = torch.nn.Parameter((torch.randn(n, c, device=dev, generator=g) / c ** 0.5).bfloat16().float())
    b = torch.nn.Parameter(torch.randn(n, device=dev, generator=g) * 0.1)
    gamma = torch.nn.Parameter(1 + 0.2 * torch.randn(c, device=dev, generator=g))
    beta = torch.nn.Parameter(0.1 * torch.randn(c, device=dev, generator=g))
    stats = F3.row_stats(x)
    ref_sum = x.float().sum(1)
    assert torch.allclose(stats[:, 0], ref_sum, rtol=1e-5, atol=1e-3)
    assert torch.allclose(stats[:, 1], (x.float() ** 2).sum(1), rtol=1e-4, atol=1e-3)
    with torch.no_grad():
        fused = F3.linear_inference(x, w, b, nsplit=nsplit, epilogue=epi, ln=(gamma, beta, 1e-5), ln_stats=stats)
        y = torch.empty_like(x)
        pshattn.layernorm_bf16(x, gamma.detach(), beta.detach(), y, 1e-5)
        out_n = n // 2 if epi == 2 else n
        unfused = torch.empty((nsplit, m, out_n // nsplit) if nsplit > 1 else (m, out_n), dtype=torch.bfloat16, device=dev)
        pshattn.linear_bf16(y, w.detach().bfloat16(), b.detach(), unfused, nsplit=nsplit, epilogue=epi)
        pshattn.device_status()
        z = torch.nn.functional.layer_norm(x.float(), (c,), gamma, beta, 1e-5) @ w.t() + b
        if epi == 2:
            z = torch.nn.functional.silu(z[:, :n // 2]) * z[:, n // 2:]
        if nsplit > 1:
            z = torch.stack(z.chunk(nsplit, dim=1))
    # the SwiGLU output is a product of two columns that each carry a rounding error: twice the plain bars
    _check(fused, z, f"ln_fold_c{c}_n{n}_epi{epi}", max_abs=4e-2 if epi == 2 else 2e-2, mean_rel=2e-3 if epi == 2 else 1e-3)
    # and the fused result is as close to fp32 as the unfused pair is (which rounds the normalised rows to bf16 first)
    e_f = (fused.float() - z).abs().mean().item()
    e_u = (unfused.float() - z).abs().mean().item()
    assert e_f <= 1.25 * e_u + 1e-6, (e_f, e_u)


@pytest.mark.parametrize("m,k,n", [(3000, 32, 32), (2048, 256, 64), (999, 128, 128), (1024, 2048, 512), (40000, 64, 256),
                                   (30000, 512, 512)])
def test_row_sums_from_the_epilogue(cuda_device, m, k, n):
    from flash3dtransformer_b200.layers import functional as F3
    dev = cuda_device
    g = torch.Generator(dev).manual_seed(k)
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w = torch.nn.Parameter(torch.randn(n, k, device=dev, generator=g) / k ** 0.5)
    b = torch.nn.Parameter(torch.randn(n, device=dev, generator=g))
    res = torch.randn(m, n, device=dev, generator=g).bfloat16()
    with torch.no_grad():
        out, stats = F3.linear_inference(x, w, b, residual=res, want_stats=True)
        for _ in range(3):                                     # the sums are added in a fixed order: same bits every run
            out2, stats2 = F3.linear_inference(x, w, b, residual=res, want_stats=True)
            assert torch.equal(stats, stats2) and torch.equal(out, out2)
    exact = x.float() @ w.detach().bfloat16().float().t() + b.detach() + res.float()
    # the sums are taken before the output is rounded to bf16: compare with the unrounded result
    assert torch.allclose(stats[:, 0], exact.sum(1), rtol=1e-4, atol=2e-2)
    assert torch.allclose(stats[:, 1], (exact ** 2).sum(1), rtol=2e-4, atol=2e-2)
    # and they serve as LayerNorm statistics of the stored rows
    mean_s, mean_o = stats[:, 0] / n, out.float().mean(1)
    assert (mean_s - mean_o).abs().max().item() <= 4e-3 * max(1.0, mean_o.abs().max().item())


def test_block_and_backbone_folded_against_unfused(cuda_device):
    from flash3dtransformer_b200 import configs, layers
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import bucket_scope
    dev = cuda_device
    torch.manual_seed(3)
    c, heads, bucket, k = 256, 8, 256, 2
    n = bucket * k * 4
    blk = layers.XFMR(c, 4 * c, heads, bucket, True, bucket_scope.SwinPlan("swin", bucket, k, 0), torch.nn.LayerNorm).to(dev)
    with torch.no_grad():
        for p in (blk.norm.weight, blk.mlp.mlp.layer_norm_weight):
            p.add_(0.2 * torch.randn_like(p))
        for p in (blk.norm.bias, blk.mlp.mlp.layer_norm_bias):
            p.add_(0.1 * torch.randn_like(p))
    x = (torch.randn(n, c, device=dev) * 2 + 0.5).bfloat16()
    with torch.no_grad():
        folded = blk(None, x, None)
        assert hasattr(folded, "_f3d_row_stats")
    with torch.enable_grad():                                  # the unfused path is the one that autograd uses
        unfused = blk(None, x.clone().requires_grad_(True), None).detach()
    _check(folded, unfused.float(), "xfmr_block_folded_vs_unfused", max_abs=6e-2, mean_rel=4e-3)
    # whole backbone: folded (no_grad) against unfused (grad mode), same weights and input
    model = configs.flash3d_backbone(channels=(64, 256), depths=(2, 2)).to(dev)       # the deeper level folds
    c32, seps = synthetic.batch(synthetic.lidar_scan, [30000, 22000], seed=4)
    coords = torch.from_numpy(c32.astype(np.float16)).to(dev)
    sp = torch.from_numpy(seps.astype(np.uint32)).to(dev)
    launches0 = pshattn.launch_count()
    with torch.no_grad():
        a = model(coords, None, sp)
    folded_launches = pshattn.launch_count() - launches0
    launches0 = pshattn.launch_count()
    with torch.enable_grad():
        b = model(coords, None, sp).detach()
    unfused_launches = pshattn.launch_count() - launches0
    pshattn.device_status()
    rows = int(seps[-1])
    _check(a[:rows], b[:rows].float(), "backbone_folded_vs_unfused", max_abs=0.1, mean_rel=1e-2)
    assert folded_launches < unfused_launches            # 8 LayerNorm launches gone, 2 statistics passes added
