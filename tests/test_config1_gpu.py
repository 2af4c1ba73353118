"""The CPU-runnable configuration end to end on the GPU: one synthetic scan of 20,000 points (70 % ground plane, 30 %
Gaussian blobs), PSH bucketing at bucket size 256 (128 buckets, 20,224 padded rows = 79 buckets of tokens), then one
bucketed-attention layer of dim 128 = 4 heads x 32 on fp16 features ~N(0,1) with default nn.Linear initialisation,
seed 0: QKV projection, attention over each bucket, output projection.

Bars: bucket ids, offsets, counters and scattered coordinates bit-exact against the CPU oracle; the layer output against
an fp32 evaluation of the same layer from the same fp16 inputs, max abs <= 2e-2 and mean |err| / mean |ref| <= 1e-3 as
raw numbers for fp16 (what was measured on a B200 is appended to gpurun_out/parity_achieved.jsonl); for bf16 the mean bar
is applied above the floor that rounding the exact output to bf16 sets, as in the other tests."""
import numpy as np
import pytest
import torch

from conftest import record_parity
from flash3dtransformer_b200 import synthetic
from oracle import attn_oracle as ao
from oracle import psh_oracle as po

pytestmark = pytest.mark.gpu

N, BUCKET, C, H, D = 20000, 256, 128, 4, 32


def _layer_reference(x, wqkv, bqkv, wp, bp, l, scopes):
    """fp32 evaluation from the 16-bit inputs, nothing rounded in between."""
    qkv = x.float() @ wqkv.float().t() + bqkv
    q, k, v = (t.reshape(1, l, H, D) for t in qkv.chunk(3, dim=-1))
    o, _ = ao.buck_swin_fwd(q, k, v, scopes, BUCKET)
    return o.reshape(l, C) @ wp.float().t() + bp


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cpu_runnable_configuration(cuda_device, dtype, scope=1):
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import psh_main
    dev = cuda_device
    c32, seps = synthetic.batch(synthetic.ground_and_blobs, [N], seed=0)
    c16 = c32.astype(np.float16)
    pad_to = -(-N // BUCKET) * BUCKET
    assert pad_to == 20224
    # ---- PSH: bit-exact
    scattered, buf = psh_main.batch_bucket_scatter(torch.from_numpy(c16).to(dev), torch.from_numpy(seps.astype(np.uint32)).to(dev),
                                                   BUCKET, pad_to, 2)
    nb, div = po.psh_params([N], BUCKET)
    assert (nb, div) == (128, 512)
    ref = po.psh_scatter(c16, seps, nb, div, BUCKET, 0xFFFF, c16.min(0), c16.max(0), po.probe_table(), pad_to, 0.0, 2)
    assert np.array_equal(buf.bucket_id.cpu().numpy(), ref["bucket_id"])
    assert np.array_equal(buf.bucket_offs.cpu().numpy(), ref["bucket_offs"])
    assert np.array_equal(buf.bucket_cntr.cpu().numpy(), ref["bucket_cntr"])
    assert np.array_equal(scattered.cpu().numpy().view(np.uint16), ref["scattered_coord"].view(np.uint16))
    # ---- the attention layer on features of the bucket-ordered rows
    torch.manual_seed(0)
    l = pad_to
    x = torch.randn(l, C).to(dtype)
    qkv_lin, proj_lin = torch.nn.Linear(C, 3 * C), torch.nn.Linear(C, C)
    wqkv, wp = qkv_lin.weight.detach().to(dtype), proj_lin.weight.detach().to(dtype)
    bqkv, bp = qkv_lin.bias.detach().float(), proj_lin.bias.detach().float()
    # every bucket attends to itself (the layer as configured: 79 buckets of 256 tokens)
    scopes = torch.arange(l // BUCKET, dtype=torch.int64).reshape(-1, scope)
    qkv = torch.empty(3, l, C, dtype=dtype, device=dev)
    pshattn.linear_bf16(x.to(dev), wqkv.to(dev), bqkv.to(dev), qkv, nsplit=3)
    q, k, v = (qkv[i].view(1, l, H, D) for i in range(3))
    o = torch.empty(1, l, H, D, dtype=dtype, device=dev)
    lse = torch.zeros(1, l, H, device=dev)
    pshattn.buck_swin_fwd(q, k, v, o, lse, scopes.to(torch.uint32).to(dev), BUCKET)
    out = torch.empty(l, C, dtype=dtype, device=dev)
    pshattn.linear_bf16(o.view(l, C), wp.to(dev), bp.to(dev), out)
    pshattn.device_status()
    want = _layer_reference(x, wqkv, bqkv, wp, bp, l, scopes)
    got = out.float().cpu()
    err = (got - want).abs()
    max_abs = err.max().item()
    mean_rel = (err.mean() / want.abs().mean()).item()
    floor = ((want.to(dtype).float() - want).abs().mean() / want.abs().mean()).item()
    record_parity(f"config1_layer_{str(dtype).split('.')[-1]}_scope{scope}", max_abs_raw=max_abs, mean_rel_raw=mean_rel,
                  rounding_floor=floor, ref_abs_max=want.abs().max().item(), bound_max_abs=2e-2, bound_mean_rel=1e-3)
    assert torch.isfinite(got).all()
    assert max_abs <= 2e-2, max_abs
    if dtype == torch.float16:
        assert mean_rel <= 1e-3, mean_rel                      # the stated bar, as raw numbers
    else:
        assert mean_rel <= floor + 1e-3, (mean_rel, floor)     # a bf16 output cannot be nearer than its own rounding
