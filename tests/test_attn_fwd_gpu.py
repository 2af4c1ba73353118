"""GPU parity of bucketed attention forward against the fp32 CPU oracle.  Tolerance on N(0,1) bf16 inputs:
max abs <= 2e-2 against the fp32 oracle; mean|err| / mean|ref| exceeds the floor set by rounding the exact result to
bf16 (about 1.4e-3) by at most 1e-3; LSE max abs <= 2e-2.  Shapes follow the reference's tests
(tests/test_attn_fwd.py:295-452): (B,L,H,D) = (3,1280,2,128)/bucket 256, (16,4096,4,16)/512, (8,1280,2,128)/256."""
import pytest
import torch

from conftest import record_parity
from oracle import attn_oracle as ao

pytestmark = pytest.mark.gpu


def _run(dev, b, l, h, d, bucket, scopes, mul=1.0, seed=0):
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(b, l, h, d, generator=g) * mul).bfloat16() for _ in range(3))
    sc = torch.tensor(scopes, dtype=torch.int64)
    o = torch.zeros(b, l, h, d, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(b, l, h, dtype=torch.float32, device=dev)
    pshattn.buck_swin_fwd(q.to(dev), k.to(dev), v.to(dev), o, lse, sc.to(torch.uint32).to(dev), bucket)
    pshattn.device_status()
    ref_o, ref_lse = ao.buck_swin_fwd(q, k, v, sc, bucket)
    return o.float().cpu(), lse.cpu(), ref_o, ref_lse


def _check(o, lse, ref_o, ref_lse, max_abs=2e-2, mean_rel=1e-3):
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    err = (o - ref_o).abs() / ref_o.abs().clamp(min=1.0)
    rel = ((o - ref_o).abs().mean() / ref_o.abs().mean()).item()
    floor = ((ref_o.bfloat16().float() - ref_o).abs().mean() / ref_o.abs().mean()).item()
    record_parity("attn_fwd", max_abs_raw=(o - ref_o).abs().max().item(), max_abs_scaled=err.max().item(), mean_rel_raw=rel,
                  rounding_floor=floor, lse_max_abs=(lse - ref_lse).abs().max().item(), ref_abs_max=ref_o.abs().max().item(),
                  bound_max_abs=max_abs, bound_mean_rel_excess=mean_rel)
    assert err.max().item() <= max_abs, f"O max abs {err.max().item()}"
    assert rel <= floor + mean_rel, f"O mean rel {rel} (bf16 rounding floor {floor})"
    assert (lse - ref_lse).abs().max().item() <= max_abs, f"LSE max abs {(lse - ref_lse).abs().max().item()}"


@pytest.mark.parametrize("d", [16, 32, 64, 128])
def test_single_bucket_scopes(cuda_device, d):
    # 4 buckets of 256 tokens, every bucket its own scope
    _check(*_run(cuda_device, 2, 1024, 2, d, 256, [[0], [1], [2], [3]]))


@pytest.mark.parametrize("b,l,h,d,bucket,k", [(3, 1280, 2, 128, 256, 5), (2, 4096, 4, 16, 512, 4), (1, 4096, 4, 32, 512, 8),
                                             (2, 2048, 8, 32, 512, 2), (1, 1536, 2, 64, 128, 3)])
def test_multi_bucket_scopes(cuda_device, b, l, h, d, bucket, k):
    nb = l // bucket
    scopes = [list(range(i, i + k)) for i in range(0, nb, k)]
    _check(*_run(cuda_device, b, l, h, d, bucket, scopes, seed=1))


def test_permuted_buckets_inside_scope_and_unlisted_buckets(cuda_device):
    """The result does not depend on the order of the buckets inside a scope (tests/test_attn_fwd.py:418-452);
    buckets that no scope lists keep the caller's O."""
    a = _run(cuda_device, 1, 2048, 2, 32, 256, [[0, 1, 2, 3], [4, 5, 6, 7]], seed=3)
    b = _run(cuda_device, 1, 2048, 2, 32, 256, [[3, 1, 0, 2], [6, 7, 5, 4]], seed=3)
    _check(*a)
    assert torch.allclose(a[0], b[0], atol=1e-2) and torch.allclose(a[1], b[1], atol=1e-3)
    o, lse, ref_o, ref_lse = _run(cuda_device, 1, 2048, 2, 32, 256, [[0, 5], [2, 7]], seed=4)
    _check(o, lse, ref_o, ref_lse)
    for bk in (1, 3, 4, 6):
        assert torch.all(o[:, bk * 256:(bk + 1) * 256] == 0) and torch.all(lse[:, bk * 256:(bk + 1) * 256] == 0)


@pytest.mark.parametrize("mul", [2.0, 4.0, 16.0])
def test_scaled_inputs(cuda_device, mul):
    """Inputs scaled as in the reference's tests (x2 .. x16): the softmax becomes nearly one-hot.  The reference
    accepts max < 0.3-0.6 and mean < 0.01-0.02 against SDPA (tests/test_attn_fwd.py:319-368); the same bounds are
    used here relative to the input scale."""
    o, lse, ref_o, ref_lse = _run(cuda_device, 1, 1024, 2, 32, 256, [[0, 1], [2, 3]], mul=mul, seed=5)
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    assert (o - ref_o).abs().max().item() <= 0.3 * mul / 2
    assert (o - ref_o).abs().mean().item() <= 0.01 * mul / 2
    assert ((lse - ref_lse).abs() / ref_lse.abs().clamp(min=1)).max().item() <= 2e-2


def test_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    dev = cuda_device
    q = torch.zeros(1, 512, 2, 32, dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(1, 512, 2, device=dev)
    sc = torch.zeros(1, 1, dtype=torch.uint32, device=dev)
    with pytest.raises(RuntimeError, match="multiple"):
        pshattn.buck_swin_fwd(q, q, q, q.clone(), lse, sc, 96)
    with pytest.raises(RuntimeError, match="head_dim"):
        q2 = torch.zeros(1, 512, 2, 24, dtype=torch.bfloat16, device=dev)
        pshattn.buck_swin_fwd(q2, q2, q2, q2.clone(), lse, sc, 256)
    with pytest.raises(RuntimeError, match="dtype"):
        pshattn.buck_swin_fwd(q.float(), q, q, q, lse, sc, 256)
    with pytest.raises(RuntimeError, match="four axes"):
        pshattn.buck_swin_fwd(q[0], q[0], q[0], q[0], lse, sc, 256)
