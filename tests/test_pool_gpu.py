"""GPU parity of sub-bucket construction, pooling and unpooling (forward + backward) against the CPU oracle.
Index outputs are bit-exact; feature outputs are bit-exact too because kernel and oracle accumulate in fp32 in
the same order and round once (the stated bar is 1e-5 relative for sums)."""
import numpy as np
import pytest
import torch

from oracle import pool_oracle as pl
from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu

TORCH_DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def _to_dev(x32, dtype, dev):
    return torch.from_numpy(x32).to(dev).to(TORCH_DT[dtype])


def _build(dev, c16, seps, S, feat32, dtype, op, align=1, hash_type=1):
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import subbuck as sbm
    coords = torch.from_numpy(c16).to(dev)
    feat = _to_dev(feat32, dtype, dev)
    sp = torch.from_numpy(np.asarray(seps, dtype=np.uint32)).to(dev)
    sb = sbm.SubbuckBuffers.create_subbuck_buff(coords, feat, sp, S, out_alignment=align)
    sizes = np.diff(np.concatenate([[0], seps]))
    pshattn.batch_subbuck_reduce(coords, feat, sp, int(sizes.max()), S, 0xFFFF, sb.bbox_min, sb.bbox_max,
                                 sb.subbuck_id, sb.subbuck_off, sb.reduced_sep, sb.reduced_coord, sb.reduced_feat,
                                 sb.unpool_ind, hash_type, op)
    torch.cuda.synchronize()
    return coords, feat, sb


@pytest.mark.parametrize("S,dtype,op", [(2, "bf16", 0), (2, "fp32", 1), (3, "bf16", 2), (4, "fp16", 3), (2, "bf16", 3)])
def test_subbuck_and_reduce_bit_exact(cuda_device, S, dtype, op):
    c32, seps = synthetic.batch(synthetic.lidar_scan, [5000, 1, 1025, 2048, 777, 3333], seed=1)
    c16 = c32.astype(np.float16)
    n = c16.shape[0]
    C = 64
    feat32 = pl._round(np.random.default_rng(0).normal(size=(n + 40, C)).astype(np.float32), dtype)
    coords, feat, sb = _build(cuda_device, c16, seps, S, feat32, dtype, op, align=256)
    sid, soff, unpool, rcoord, red_sep = pl.subbuck_build(c16, seps, S, red_rows_aligned=sb.reduced_coord.shape[0])
    assert np.array_equal(sb.reduced_sep.cpu().numpy().astype(np.int64), red_sep)
    assert np.array_equal(sb.subbuck_id.cpu().numpy(), sid)
    assert np.array_equal(sb.subbuck_off.cpu().numpy(), soff)
    assert np.array_equal(sb.unpool_ind.cpu().numpy(), unpool)
    assert np.array_equal(sb.reduced_coord.cpu().numpy().view(np.uint16), rcoord.view(np.uint16))
    pl.subbuck_invariants(sid, soff, sb.unpool_ind.cpu().numpy(), sb.reduced_coord.cpu().numpy(), c16, seps, S)
    exp = pl.pool_reduce(feat32, unpool, n, op, sb.reduced_feat.shape[0], dtype)
    got = sb.reduced_feat.float().cpu().numpy()
    assert np.array_equal(got, exp), f"max diff {np.abs(got - exp).max()}"


@pytest.mark.parametrize("dtype,op,S", [("bf16", 0, 2), ("bf16", 1, 2), ("fp32", 2, 4), ("bf16", 3, 4), ("fp16", 0, 3)])
def test_reduce_backward(cuda_device, dtype, op, S):
    from flash3dtransformer_b200.lib import pshattn
    c32, seps = synthetic.batch(synthetic.lidar_scan, [4000, 2500], seed=4)
    c16 = c32.astype(np.float16)
    n = c16.shape[0]
    C = 128
    rng = np.random.default_rng(1)
    feat32 = pl._round(rng.normal(size=(n, C)).astype(np.float32), dtype)
    coords, feat, sb = _build(cuda_device, c16, seps, S, feat32, dtype, op)
    unpool = sb.unpool_ind.cpu().numpy()
    g32 = pl._round(rng.normal(size=(unpool.shape[0], C)).astype(np.float32), dtype)
    g = _to_dev(g32, dtype, cuda_device)
    gin = torch.zeros_like(feat)
    pshattn.batch_subbuck_reduce_backward(g, feat, sb.unpool_ind, gin, S, op)
    torch.cuda.synchronize()
    exp = pl.pool_reduce_bwd(g32, feat32, unpool, n, op, dtype)
    assert np.array_equal(gin.float().cpu().numpy(), exp)


@pytest.mark.parametrize("dtype,C", [("bf16", 32), ("bf16", 256), ("fp32", 128), ("fp16", 8)])
def test_unpool_forward_backward(cuda_device, dtype, C):
    from flash3dtransformer_b200.lib import pshattn
    c32, seps = synthetic.batch(synthetic.lidar_scan, [3000, 1500, 20], seed=7)
    c16 = c32.astype(np.float16)
    n = c16.shape[0]
    rng = np.random.default_rng(2)
    S = 2
    feat32 = pl._round(rng.normal(size=(n + 100, C)).astype(np.float32), dtype)
    coords, feat, sb = _build(cuda_device, c16, seps, S, feat32, dtype, 0, align=64)
    unpool = sb.unpool_ind.cpu().numpy()
    down32 = pl._round(rng.normal(size=(sb.reduced_feat.shape[0], C)).astype(np.float32), dtype)
    down = _to_dev(down32, dtype, cuda_device)
    up = torch.full_like(feat, float("nan"))
    pshattn.additive_unpool_fwd(feat, down, up, sb.unpool_ind, S, covered_rows=n)
    torch.cuda.synchronize()
    exp = pl.unpool_add(feat32, down32, unpool, dtype)
    assert np.array_equal(up.float().cpu().numpy(), exp)
    # reference behaviour: rows behind the pooled range stay untouched
    up2 = torch.full_like(feat, 7.0)
    pshattn.additive_unpool_fwd(feat, down, up2, sb.unpool_ind, S)
    assert torch.all(up2[n:] == 7.0) and torch.equal(up2[:n], up[:n])
    g32 = pl._round(rng.normal(size=feat32.shape).astype(np.float32), dtype)
    g = _to_dev(g32, dtype, cuda_device)
    g_res = torch.zeros_like(g)
    g_down = torch.zeros_like(down)
    pshattn.additive_unpool_bwd(g_res, g_down, g, sb.unpool_ind, S)
    torch.cuda.synchronize()
    e_res, e_down = pl.unpool_add_bwd(g32, unpool, down32.shape[0], dtype)
    assert np.array_equal(g_res.float().cpu().numpy(), e_res)
    assert np.array_equal(g_down.float().cpu().numpy(), e_down)


def test_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    t = torch.zeros(16, 8, dtype=torch.bfloat16, device=cuda_device)
    ind = torch.zeros(8, 2, dtype=torch.uint32, device=cuda_device)
    with pytest.raises(RuntimeError, match="subbucket_size"):
        pshattn.additive_unpool_fwd(t, t, t.clone(), ind, 3)
    with pytest.raises(RuntimeError, match="contiguous"):
        pshattn.additive_unpool_fwd(t[:, ::2], t, t, ind, 2)
    with pytest.raises(RuntimeError, match="16 bytes"):
        pshattn.additive_unpool_fwd(t[:, :4].contiguous(), t[:, :4].contiguous(), t[:, :4].contiguous(), ind, 2)
    with pytest.raises(RuntimeError, match="reduction"):
        pshattn.batch_subbuck_reduce_backward(t[:8].contiguous(), t, ind, t.clone(), 2, 9)


def test_full_size_pool_unpool_properties(cuda_device):
    """1,000,000-point heavy-tailed scene, C=128 fp32, three rounds of stride-2 pooling and the matching unpools:
    sum pooling preserves the column sums (1e-5 relative) and unpooling a zero residual replicates rows."""
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import subbuck as sbm
    dev = cuda_device
    c32, seps = synthetic.batch(synthetic.zipf_voxels, [1_000_000], seed=0)
    coords = torch.from_numpy(c32.astype(np.float16)).to(dev)
    sp = torch.from_numpy(seps.astype(np.uint32)).to(dev)
    feat = torch.randn(coords.shape[0], 128, device=dev, generator=torch.Generator(dev).manual_seed(0))
    col0 = feat.double().sum(0)
    levels = []
    for _ in range(3):
        sb = sbm.SubbuckBuffers.create_subbuck_buff(coords, feat, sp, 2)
        n = int(sbm.calc_red_sep_sizes(sp, 1)[0])
        pshattn.batch_subbuck_reduce(coords, feat, sp, n, 2, 0xFFFF, sb.bbox_min, sb.bbox_max, sb.subbuck_id,
                                     sb.subbuck_off, sb.reduced_sep, sb.reduced_coord, sb.reduced_feat, sb.unpool_ind,
                                     1, 1)
        ind = sb.unpool_ind.to(torch.int64)
        flat = ind[ind < coords.shape[0]]
        assert flat.numel() == coords.shape[0] and torch.equal(torch.sort(flat)[0], torch.arange(coords.shape[0], device=dev))
        col = sb.reduced_feat.double().sum(0)
        assert torch.allclose(col, col0, rtol=1e-5, atol=1e-3)
        levels.append((feat, sb))
        coords, feat, sp = sb.reduced_coord, sb.reduced_feat, sb.reduced_sep
    down = feat
    for res, sb in reversed(levels):
        up = torch.empty_like(res)
        pshattn.additive_unpool_fwd(torch.zeros_like(res), down, up, sb.unpool_ind, 2)
        down = up
    # every original row now carries the sum of its 8-point (or smaller) group: column sums scale accordingly
    assert torch.isfinite(down).all()
    ind = levels[0][1].unpool_ind.to(torch.int64)
    first = ind[:, 0]
    second = ind[:, 1]
    ok = second < down.shape[0]
    assert torch.equal(down[first[ok]], down[second[ok]])
