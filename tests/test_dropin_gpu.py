"""The drop-in claim, shown on a GPU: the reference's own, unmodified host code runs on this library.

`flash3dtransformer_b200.compat.install` imports the reference's `flash3dxfmr` Python package from a reference checkout
($F3D_REFERENCE) with `compat/flash3dxfmr/lib/pshattn.py` where the reference's build would put its compiled extension.
The tests then call the reference's host functions - `psh_main.batch_bucket_scatter` (flash3dxfmr/psh/psh_main.py:70-125),
`pooling.SubbuckReduceFunction` (layers/pooling.py:20-116), `unpool.AdditiveUnpoolFunction` (layers/unpool.py:18-77),
`buck_swin.BuckSwinFwdFunction` (layers/buck_swin.py:20-95) forward and backward, and the whole `Flash3D` model of the
reference's integration test (tests/test_psh_hourglass.py:51-163) - and compare with this repository's own layers: bit for
bit for the operators, within the bf16 bar for the model (the reference's layers run their projections on the library
GEMM and add residuals separately, this repository's layers fuse them).

Skipped where no reference checkout is given: the library itself never reads one.
"""
import os
import random

import numpy as np
import pytest
import torch

from conftest import record_parity
from flash3dtransformer_b200 import compat, synthetic

pytestmark = pytest.mark.gpu

REF = os.environ.get("F3D_REFERENCE", "")


@pytest.fixture(scope="module")
def ref(cuda_device):
    if not REF or not os.path.isdir(os.path.join(REF, "flash3dxfmr")):
        pytest.skip("set F3D_REFERENCE to a reference checkout to run the reference's host code on this library")
    pkg = compat.install(REF)
    yield pkg
    compat.uninstall()


def _batch(dev, sizes, seed=0):
    c32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=seed)
    return torch.from_numpy(c32.astype(np.float16)).to(dev), torch.from_numpy(seps.astype(np.uint32)).to(dev)


def _bits(t):
    return t.contiguous().view(torch.uint8)


def _same(a, b):
    return a.shape == b.shape and a.dtype == b.dtype and torch.equal(_bits(a), _bits(b))


def test_reference_psh_host_code(ref, cuda_device, monkeypatch):
    from flash3dxfmr.psh import psh_main as ref_pm
    from flash3dtransformer_b200.psh import psh_main as our_pm
    # the reference shuffles the probe table with Python's global generator on every call (psh/bucket.py:35); with
    # the shuffle switched off its table is in generation order, which is the fixed order this repository uses
    monkeypatch.setattr(random, "shuffle", lambda rows: None)
    coords, seps = _batch(cuda_device, [30000, 22000, 41000])
    for hash_op in (1, 2, 3, 4):
        pad_to = -(-coords.shape[0] // 512) * 512
        r_sc, r_buf = ref_pm.batch_bucket_scatter(coords, seps, 512, pad_to, hash_op)
        o_sc, o_buf = our_pm.batch_bucket_scatter(coords, seps, 512, pad_to, hash_op)
        assert _same(r_buf.probe_offs, o_buf.probe_offs)
        for name in ("bucket_id", "bucket_cntr", "bucket_offs", "bucket_cumsum", "scattered_coord"):
            assert _same(getattr(r_buf, name), getattr(o_buf, name)), (hash_op, name)
        assert _same(r_sc, o_sc) and not torch.isnan(r_sc).any()
        # the verification block of the reference's own PSH test, tests/test_psh.py:109-129
        from flash3dxfmr.lib import pshattn
        cntr = r_buf.bucket_cntr
        offset_maxcnt, _ = torch.max(cntr.to(torch.int32), dim=-1)
        offset_maxcnt = offset_maxcnt.to(torch.uint32)
        max_cntr = int(torch.max(cntr.to(torch.int32)))
        table = torch.zeros((seps.shape[0], cntr.shape[1], max_cntr), dtype=torch.int8, device=cuda_device)
        res = cntr.detach().clone()
        assert torch.all(torch.cumsum(cntr.to(torch.int64), dim=1) == r_buf.bucket_cumsum.to(torch.int64))
        pshattn.batch_bucket_sanitizer_cpu(r_buf.bucket_id, cntr, r_buf.bucket_offs, table, res, seps, offset_maxcnt,
                                           seps.shape[0], cntr.shape[1])
        assert int(res.to(torch.int64).sum()) == 0 and int(table.to(torch.int64).sum()) == coords.shape[0]


def test_reference_pooling_and_unpooling_host_code(ref, cuda_device):
    from flash3dxfmr.layers import pooling as ref_pool, unpool as ref_unpool
    from flash3dtransformer_b200.layers import pooling as our_pool, unpool as our_unpool
    from flash3dtransformer_b200.psh import psh_main as our_pm
    coords, seps = _batch(cuda_device, [9000, 12000], seed=3)
    n = coords.shape[0]
    scattered, _ = our_pm.batch_bucket_scatter(coords, seps, 512, n, 2)
    torch.manual_seed(0)
    feat = torch.randn(n, 64, device=cuda_device).bfloat16()
    for red_op in (0, 1, 2, 3):
        outs = []
        for pool, unpool in ((ref_pool, ref_unpool), (our_pool, our_unpool)):
            x = feat.clone().requires_grad_(True)
            red, sb = pool.SubbuckReduceFunction.apply(scattered, x, seps, 2, red_op, 1024)
            down = (red * 0.5).detach().requires_grad_(True)
            res = feat.clone().requires_grad_(True)
            up = unpool.AdditiveUnpoolFunction.apply(res, down, sb, 2)
            g = torch.arange(up.numel(), device=cuda_device, dtype=torch.float32).view_as(up).remainder(7.0).bfloat16()
            up.backward(g)
            red.backward(torch.ones_like(red))
            outs.append((red.detach(), sb.reduced_coord, sb.unpool_ind, sb.reduced_sep, up.detach(), x.grad, down.grad, res.grad))
        # rows behind the pooled range of `up` are not written by the reference's host code (torch.empty): compare the
        # rows an index refers to, everything else bit for bit
        names = ("reduced_feat", "reduced_coord", "unpool_ind", "reduced_sep", "up", "grad_input", "grad_down", "grad_res")
        for name, a, b in zip(names, *outs):
            rows = slice(0, int(seps[-1].item())) if name == "up" else slice(None)
            assert _same(a[rows], b[rows]), (red_op, name)


def test_reference_attention_host_code(ref, cuda_device):
    from flash3dxfmr.layers import buck_swin as ref_bs
    from flash3dxfmr.psh import bucket_scope as ref_scope
    from flash3dtransformer_b200.layers import buck_swin as our_bs
    torch.manual_seed(1)
    bucket, k, h, d = 256, 2, 4, 32            # 512-token windows: the backward kernel without atomics, same bits every run
    l = bucket * k * 6
    scopes = ref_scope.SwinPlan("swin", bucket, k, 0).gen_scopes_from_plan(l, cuda_device)
    base = [torch.randn(1, l, h, d, device=cuda_device).bfloat16() for _ in range(3)]
    g = torch.randn(1, l, h, d, device=cuda_device).bfloat16()
    outs = []
    for mod in (ref_bs, our_bs):
        q, kk, v = (t.clone().requires_grad_(True) for t in base)
        o = mod.BuckSwinFwdFunction.apply(q, kk, v, scopes, bucket)
        o.backward(g)
        outs.append((o.detach(), q.grad, kk.grad, v.grad))
    for name, a, b in zip(("O", "dQ", "dK", "dV"), *outs):
        assert _same(a, b), name
    # and against fp32 softmax attention over each scope
    qf, kf, vf = (t.float().view(l // (bucket * k), bucket * k, h, d).transpose(1, 2) for t in base)
    want = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf).transpose(1, 2).reshape(1, l, h, d)
    assert (outs[0][0].float() - want).abs().max().item() <= 2e-2


def test_reference_model_host_code(ref, cuda_device, monkeypatch):
    """The model of the reference's integration test (two levels, te.LayerNorm blocks, BatchNorm1d + GELU wrappers,
    autocast to bf16), built by the reference's own `Flash3D`, forward and backward; the same weights in this
    repository's `Flash3D` give the same features within the bf16 bar."""
    from functools import partial
    import transformer_engine.pytorch as te
    from torch import nn
    from flash3dxfmr import layers as ref_layers
    from flash3dxfmr.psh import bucket_scope as ref_scope
    from flash3dtransformer_b200 import layers as our_layers
    from flash3dtransformer_b200.psh import bucket_scope as our_scope
    from flash3dtransformer_b200.lib import pshattn

    monkeypatch.setattr(random, "shuffle", lambda rows: None)      # probe table in generation order, as above
    bucket_size, scope = 512, 8

    def specs(L, S, norm):
        def x(c, hid, heads, plan, i):
            return L.XFMRSpecs(channels=c, hid_channels=hid, num_heads=heads, qkv_bias=True,
                               swin_plan=S.SwinPlan(plan, bucket_size, scope, i), norm_layer=norm)
        wrap = dict(reduction_op="mean", pool_align=S.swinable_alignment(bucket_size, scope),
                    pool_norm=partial(nn.BatchNorm1d, eps=1e-3, momentum=0.01), pool_act=nn.GELU,
                    unpool_norm=partial(nn.BatchNorm1d, eps=1e-3, momentum=0.01), unpool_act=nn.GELU)
        return [L.F3DLevelSpecs(encoder_specs=[x(32, 128, 2, "stride", 1), x(32, 128, 2, "swin", 2)],
                                decoder_specs=[x(64, 256, 4, "swin", 3), x(64, 256, 4, "swin", 4)], **wrap),
                L.F3DLevelSpecs(encoder_specs=[x(64, 128, 4, "swin", 1), x(64, 128, 4, "swin", 2)],
                                decoder_specs=[x(64, 256, 4, "swin", 3), x(64, 256, 4, "swin", 4)], **wrap)]

    torch.manual_seed(0)
    ref_model = ref_layers.Flash3D(specs(ref_layers, ref_scope, te.LayerNorm), bucket_size, scope, 2).to(cuda_device)
    our_model = our_layers.Flash3D(specs(our_layers, our_scope, nn.LayerNorm), bucket_size, scope, 2).to(cuda_device)
    assert sorted(ref_model.state_dict()) == sorted(our_model.state_dict())
    our_model.load_state_dict(ref_model.state_dict())
    coords, seps = _batch(cuda_device, [30000, 26000], seed=5)

    feats = []
    for model in (ref_model, our_model):
        with torch.autocast(dtype=torch.bfloat16, device_type="cuda"):
            feat = model(coords, coords, seps)
            loss = feat.float().mean()
        loss.backward()
        feats.append(feat.detach().float())
        grads = [p.grad for p in model.parameters()]
        assert all(g is not None and torch.isfinite(g).all() for g in grads)
    pshattn.device_status()
    a, b = feats
    assert a.shape == b.shape and torch.isfinite(a).all()
    n = int(seps[-1].item())
    # bucket order is identical in both (same kernels, same table), so rows correspond one to one
    # not bit for bit: the reference's embedding layer rounds the fp16 coordinates to bf16 before its 3 -> C projection
    # (flash3dxfmr/layers/psh_ops.py:67; 8 mantissa bits: 0.25 m at 80 m range) where this repository's layer keeps
    # fp16, and eight transformer blocks with BatchNorm wrappers sit behind it
    err = (a[:n] - b[:n]).abs()
    scaled = (err / b[:n].abs().clamp(min=1.0)).max().item()
    mean_rel = (err.mean() / b[:n].abs().mean()).item()
    record_parity("reference_model_vs_this_repository", max_abs_scaled=scaled, mean_rel_raw=mean_rel,
                  ref_abs_max=b[:n].abs().max().item(), bound_max_abs=0.5, bound_mean_rel=2e-2)
    assert scaled <= 0.5, scaled
    assert mean_rel <= 2e-2, mean_rel
