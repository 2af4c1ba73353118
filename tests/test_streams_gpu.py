"""Calls that use the library's scratch workspace from two CUDA streams at once give the single-stream results.

The PSH tile tables, the fp32 dQ accumulator of the attention backward and the other scratch blocks are kept per
(device, stream), so work queued on different streams may overlap on the GPU without sharing scratch."""
import numpy as np
import pytest
import torch

from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu


def _psh(dev, seed, sizes):
    from flash3dtransformer_b200.psh import psh_main
    c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=seed)
    coords = torch.from_numpy(c32.astype(np.float16)).to(dev)
    sp = torch.from_numpy(seps.astype(np.uint32)).to(dev)
    return coords, sp


def test_two_streams_psh_and_attention_backward(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import psh_main
    dev = cuda_device
    inputs = [_psh(dev, 31, [60000, 45000, 52000]), _psh(dev, 32, [70000, 30000])]
    g = torch.Generator().manual_seed(3)
    l, h, d, bucket = 8192, 4, 32, 512
    attn = []
    for _ in range(2):
        q, k, v, do = (torch.randn(1, l, h, d, generator=g).bfloat16().to(dev) for _ in range(4))
        attn.append((q, k, v, do))
    sc = torch.arange(l // bucket, dtype=torch.int64).view(-1, 4).to(torch.uint32).to(dev)      # 2048-token windows: dQ through the scratch

    def work(i):
        coords, sp = inputs[i]
        n = coords.shape[0]
        _, buf = psh_main.batch_bucket_scatter(coords, sp, 512, -(-n // 512) * 512, 2)
        q, k, v, do = attn[i]
        o = torch.zeros_like(q); lse = torch.zeros(1, l, h, device=dev); delta = torch.zeros(1, l, h, device=dev)
        dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
        pshattn.buck_swin_fwd(q, k, v, o, lse, sc, bucket)
        pshattn.buck_swin_bwd(q, k, v, o, do, lse, delta, dq, dk, dv, sc, bucket)
        return buf, dq, dk, dv

    torch.cuda.synchronize()
    want = [work(0), work(1)]                       # one after the other on the current stream
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
    for rep in range(3):                            # interleaved: the calls of the two streams alternate on the host
        got = [None, None]
        for i in (0, 1):
            with torch.cuda.stream(streams[i]):
                got[i] = work(i)
        torch.cuda.synchronize()
        pshattn.device_status()
        for i in (0, 1):
            wb, wq, wk, wv = want[i]
            gb, gq, gk, gv = got[i]
            for name in ("bucket_id", "bucket_offs", "bucket_cntr", "bucket_cumsum", "scattered_coord"):
                a, b = getattr(wb, name), getattr(gb, name)
                assert torch.equal(a.view(torch.uint8), b.view(torch.uint8)), (rep, i, name)
            assert torch.equal(wk, gk) and torch.equal(wv, gv), (rep, i)
            # dQ sums fp32 partial tiles in the order the CTAs arrive: equal up to that rounding
            assert (wq.float() - gq.float()).abs().max().item() <= 2e-2 * wq.float().abs().max().item(), (rep, i)
