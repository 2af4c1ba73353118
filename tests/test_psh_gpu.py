"""GPU parity of the PSH bucketing + scatter kernels against the CPU oracle, through the operator module and the
C ABI.  Bit-exact: bucket ids, offsets, counters, cumsum and the scattered coordinates."""
import numpy as np
import pytest
import torch

from oracle import psh_oracle as po
from flash3dtransformer_b200 import synthetic

pytestmark = pytest.mark.gpu


def _gpu_scatter(dev, coords16, seps, bucket_size, hash_type, pad_to, nb=None, div=None, seed=None):
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import bucket as f3dbuck
    if seed is not None:
        pshattn.DeviceManagerSingleton.instance().set_seed(seed)
    sizes = np.diff(np.concatenate([[0], seps]))
    if nb is None:
        nb, div = po.psh_params(sizes, bucket_size)
    c = torch.from_numpy(coords16).to(dev)
    n = c.shape[0]
    b = len(seps)
    bid = torch.ones(n, dtype=torch.uint16, device=dev)
    cntr = torch.zeros(b, nb, dtype=torch.uint32, device=dev)
    offs = torch.empty(n, dtype=torch.uint32, device=dev)
    cums = torch.zeros(b, nb, dtype=torch.uint32, device=dev)
    sc = torch.full((pad_to, 3), float("nan"), dtype=torch.float16, device=dev)
    sp = torch.from_numpy(np.asarray(seps, dtype=np.uint32)).to(dev)
    probe = f3dbuck.generate_probe_offsets(dev)
    bmin = torch.from_numpy(coords16.min(0)).to(dev) if n else torch.zeros(3, dtype=torch.float16, device=dev)
    bmax = torch.from_numpy(coords16.max(0)).to(dev) if n else torch.ones(3, dtype=torch.float16, device=dev)
    pshattn.batch_psh_scatter_pad_hash(c, bid, cntr, offs, sp, int(sizes.max()) if len(sizes) else 0, nb, div,
                                       bucket_size, 0xFFFF, bmin, bmax, probe, cums, sc, 0.0, hash_type)
    torch.cuda.synchronize()
    if seed is not None:
        pshattn.DeviceManagerSingleton.instance().set_seed(3407)
    return nb, div, dict(bucket_id=bid.cpu().numpy(), bucket_offs=offs.cpu().numpy(), bucket_cntr=cntr.cpu().numpy(),
                         bucket_cumsum=cums.cpu().numpy(), scattered_coord=sc.cpu().numpy())


def _compare(out, ref):
    for k in ("bucket_cntr", "bucket_cumsum", "bucket_id", "bucket_offs"):
        assert np.array_equal(out[k], ref[k]), f"{k} differs in {np.count_nonzero(out[k] != ref[k])} places"
    assert np.array_equal(out["scattered_coord"].view(np.uint16), ref["scattered_coord"].view(np.uint16))


def _oracle(coords16, seps, nb, div, bucket_size, hash_type, pad_to, seed=3407):
    bmin = coords16.min(0) if coords16.shape[0] else np.zeros(3, np.float16)
    bmax = coords16.max(0) if coords16.shape[0] else np.ones(3, np.float16)
    return po.psh_scatter(coords16, seps, nb, div, bucket_size, 0xFFFF, bmin, bmax, po.probe_table(), pad_to, 0.0,
                          hash_type, seed)


@pytest.mark.parametrize("hash_type", [1, 2, 3, 4])
def test_cpu_runnable_config_bit_exact(cuda_device, hash_type):
    # one scan of 20,000 points, bucket 256 -> 128 buckets
    coords32, seps = synthetic.batch(synthetic.ground_and_blobs, [20000], seed=0)
    c16 = coords32.astype(np.float16)
    pad_to = -(-20000 // 256) * 256
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 256, hash_type, pad_to)
    assert nb == 128 and div == 512
    _compare(out, _oracle(c16, seps, nb, div, 256, hash_type, pad_to))
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)


@pytest.mark.parametrize("hash_type", [1, 2])
def test_lidar_batch_bit_exact(cuda_device, hash_type):
    sizes = [30000, 17001, 25013, 999]
    coords32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=5)
    c16 = coords32.astype(np.float16)
    pad_to = -(-c16.shape[0] // (512 * 6)) * 512 * 6
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 512, hash_type, pad_to)
    _compare(out, _oracle(c16, seps, nb, div, 512, hash_type, pad_to))
    assert not np.isnan(out["scattered_coord"].astype(np.float32)).any()


def test_seed_changes_only_rebalanced_points(cuda_device):
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [20000], seed=9)
    c16 = coords32.astype(np.float16)
    nb, div, a = _gpu_scatter(cuda_device, c16, seps, 256, 2, 20000, seed=1)
    _, _, b = _gpu_scatter(cuda_device, c16, seps, 256, 2, 20000, seed=1)
    _compare(a, b)                                      # same seed: same layout
    _compare(a, _oracle(c16, seps, nb, div, 256, 2, 20000, seed=1))
    _, _, c = _gpu_scatter(cuda_device, c16, seps, 256, 2, 20000, seed=2)
    po.scoreboard_check(c["bucket_id"], c["bucket_cntr"], c["bucket_offs"], seps, nb)


def test_edge_cases(cuda_device):
    pts = np.concatenate([np.random.default_rng(0).uniform(-5, 5, (700, 3)), np.zeros((1, 3)),
                          np.full((900, 3), 1.25)]).astype(np.float32)
    seps = np.array([700, 700, 701, 1601])
    c16 = pts.astype(np.float16)
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 128, 1, 1700)
    _compare(out, _oracle(c16, seps, nb, div, 128, 1, 1700))
    # odd sizes, unaligned scene starts, scenes smaller than a warp
    sizes = [31, 1, 33, 2049, 4097, 5]
    coords32, seps = synthetic.batch(synthetic.ground_and_blobs, sizes, seed=2)
    c16 = coords32.astype(np.float16)
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 64, 4, c16.shape[0] + 7)
    _compare(out, _oracle(c16, seps, nb, div, 64, 4, c16.shape[0] + 7))


def test_large_tiles_and_many_buckets(cuda_device):
    # 300k-point scene -> 6144-point tiles; 2048 buckets
    coords32, seps = synthetic.batch(synthetic.zipf_voxels, [300000, 150000], seed=1)
    c16 = coords32.astype(np.float16)
    nb, div = 2048, 32
    _, _, out = _gpu_scatter(cuda_device, c16, seps, 128, 1, c16.shape[0], nb=nb, div=div)
    _compare(out, _oracle(c16, seps, nb, div, 128, 1, c16.shape[0]))
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)


def test_argument_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    coords32, seps = synthetic.batch(synthetic.ground_and_blobs, [1000], seed=0)
    c16 = coords32.astype(np.float16)
    with pytest.raises(RuntimeError, match="bucket divisor too small"):
        _gpu_scatter(cuda_device, c16, seps, 64, 1, 1000, nb=16, div=1)
    with pytest.raises(RuntimeError, match="hash"):
        _gpu_scatter(cuda_device, c16, seps, 64, 7, 1000)
    with pytest.raises(RuntimeError, match="smaller than the input"):
        _gpu_scatter(cuda_device, c16, seps, 64, 1, 10)
    t = torch.zeros(10, 3, dtype=torch.float32, device=cuda_device)
    with pytest.raises(RuntimeError, match="dtype"):
        pshattn.batch_psh_scatter_pad_hash(t, t, t, t, t, 1, 1, 1, 1, 1, t, t, t, t, t, 0.0, 1)


def test_full_size_properties(cuda_device):
    """8 x 120,000-point scans, bucket 512 (too slow for an oracle diff in a unit test at every hash): size-
    independent properties - scoreboard, permutation checksum, cumsum, idempotence."""
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [120000] * 8, seed=0)
    c16 = coords32.astype(np.float16)
    pad_to = -(-c16.shape[0] // (512 * 6)) * 512 * 6
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 512, 2, pad_to)
    assert nb == 256
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)
    assert np.array_equal(np.cumsum(out["bucket_cntr"].astype(np.int64), 1), out["bucket_cumsum"].astype(np.int64))
    w = np.array([1, 1 << 16, 1 << 32])
    for s in range(8):
        a, b = s * 120000, (s + 1) * 120000
        assert (c16[a:b].view(np.uint16).astype(np.int64) @ w).sum() == \
               (out["scattered_coord"][a:b].view(np.uint16).astype(np.int64) @ w).sum()
    assert np.all(out["scattered_coord"][960000:] == 0)
    _, _, again = _gpu_scatter(cuda_device, c16, seps, 512, 2, pad_to)
    _compare(out, again)
    _compare(out, _oracle(c16, seps, nb, div, 512, 2, pad_to))


def test_pooling_bench_configuration_bit_exact(cuda_device):
    """The PSH + pooling configuration at its full size: 8 heavy-tailed scenes of 1,000,000 points, bucket 2048,
    Z-order hash.  Every PSH output equals the CPU oracle bit for bit (about a minute of oracle time), then the
    sub-bucket build and a stride-2 sum pooling of fp32 features on the scattered coordinates equal the pooling oracle."""
    from oracle import pool_oracle as pl
    from flash3dtransformer_b200.lib import pshattn
    from flash3dtransformer_b200.psh import subbuck as sbm
    sizes = [1_000_000] * 8
    coords32, seps = synthetic.batch(synthetic.zipf_voxels, sizes, seed=0)
    c16 = coords32.astype(np.float16)
    n = c16.shape[0]
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 2048, 1, n)
    assert nb == 512
    _compare(out, _oracle(c16, seps, nb, div, 2048, 1, n))
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)
    sc16 = out["scattered_coord"]
    C = 32
    feat32 = np.random.default_rng(1).normal(size=(n, C)).astype(np.float32)
    coords = torch.from_numpy(sc16).to(cuda_device)
    feat = torch.from_numpy(feat32).to(cuda_device)
    sp = torch.from_numpy(np.asarray(seps, dtype=np.uint32)).to(cuda_device)
    sb = sbm.SubbuckBuffers.create_subbuck_buff(coords, feat, sp, 2)
    pshattn.batch_subbuck_reduce(coords, feat, sp, max(sizes), 2, 0xFFFF, sb.bbox_min, sb.bbox_max, sb.subbuck_id,
                                 sb.subbuck_off, sb.reduced_sep, sb.reduced_coord, sb.reduced_feat, sb.unpool_ind, 1, 1)
    torch.cuda.synchronize()
    sid, soff, unpool, rcoord, red_sep = pl.subbuck_build(sc16, seps, 2, red_rows_aligned=sb.reduced_coord.shape[0])
    assert np.array_equal(sb.reduced_sep.cpu().numpy().astype(np.int64), red_sep)
    assert np.array_equal(sb.subbuck_id.cpu().numpy(), sid)
    assert np.array_equal(sb.subbuck_off.cpu().numpy(), soff)
    assert np.array_equal(sb.unpool_ind.cpu().numpy(), unpool)
    assert np.array_equal(sb.reduced_coord.cpu().numpy().view(np.uint16), rcoord.view(np.uint16))
    exp = pl.pool_reduce(feat32, unpool, n, 1, sb.reduced_feat.shape[0], "fp32")
    assert np.array_equal(sb.reduced_feat.cpu().numpy(), exp)


def test_scene_sharded_run_reproduces_full_batch(cuda_device):
    """Two 'ranks' (run one after the other on this GPU) that get the global bounding box, mean scene size and the
    global index of their first scene produce, scene by scene, the bits of the unsharded run."""
    from flash3dtransformer_b200 import parallel
    from flash3dtransformer_b200.psh import psh_main
    sizes = [9000, 7000, 11000, 5000, 6000]
    coords32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=21)
    coords = torch.from_numpy(coords32.astype(np.float16)).to(cuda_device)
    seps_t = torch.from_numpy(seps.astype(np.uint32)).to(cuda_device)
    n = coords.shape[0]
    _, full = psh_main.batch_bucket_scatter(coords, seps_t, 256, n, 2)
    (lo, hi), mean_n = parallel.global_psh_stats(coords, seps_t)
    for rank in range(2):
        local, lseps, (r0, r1), scene0 = parallel.shard_batch(coords, seps_t, rank, 2)
        _, mine = psh_main.batch_bucket_scatter(local, lseps, 256, local.shape[0], 2, bbox=(lo, hi), mean_n=mean_n,
                                                scene_base=scene0)
        assert torch.equal(mine.bucket_id, full.bucket_id[r0:r1])
        assert torch.equal(mine.bucket_offs.view(torch.int32), full.bucket_offs[r0:r1].view(torch.int32))
        assert torch.equal(mine.scattered_coord.view(torch.int16), full.scattered_coord[r0:r1].view(torch.int16))
    psh_main.f3ddev.get_dev_manager().set_scene_base(0)


def _gpu_index(dev, out, seps, pad_to, inverse=True):
    from flash3dtransformer_b200.lib import pshattn
    t = lambda k: torch.from_numpy(out[k]).to(dev)
    sp = torch.from_numpy(np.asarray(seps, dtype=np.uint32)).to(dev)
    o2i = torch.full((pad_to,), 0x7FFFFFFF, dtype=torch.uint32, device=dev)
    i2o = torch.empty(len(out["bucket_id"]), dtype=torch.uint32, device=dev) if inverse else None
    pshattn.scatter_index(t("bucket_id"), t("bucket_offs"), t("bucket_cumsum"), sp, o2i, i2o)
    torch.cuda.synchronize()
    return o2i, i2o


@pytest.mark.parametrize("sizes,bucket,pad_align", [([20000], 256, 256), ([30000, 17001, 25013, 999], 512, 512 * 6),
                                                     ([31, 1, 33, 2049, 4097, 5], 64, 7)])
def test_scatter_index_bit_exact(cuda_device, sizes, bucket, pad_align):
    coords32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=21)
    c16 = coords32.astype(np.float16)
    n = c16.shape[0]
    pad_to = -(-n // pad_align) * pad_align
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, bucket, 2, pad_to)
    ref_o2i, ref_i2o = po.scatter_index(out["bucket_id"], out["bucket_offs"], out["bucket_cumsum"], seps, pad_to)
    o2i, i2o = _gpu_index(cuda_device, out, seps, pad_to)
    assert np.array_equal(o2i.cpu().numpy(), ref_o2i) and np.array_equal(i2o.cpu().numpy(), ref_i2o)
    # the inverse index is optional
    o2i_only, none = _gpu_index(cuda_device, out, seps, pad_to, inverse=False)
    assert none is None and torch.equal(o2i_only, o2i)
    # gathering the input coordinates through out2in is the coordinate scatter, bit for bit
    from flash3dtransformer_b200.lib import pshattn
    c4 = torch.zeros(n, 4, dtype=torch.float16, device=cuda_device)          # 8-byte rows
    c4[:, :3] = torch.from_numpy(c16).to(cuda_device)
    g = torch.empty(pad_to, 4, dtype=torch.float16, device=cuda_device)
    pshattn.gather_rows(c4, o2i, g)
    assert np.array_equal(g[:, :3].cpu().numpy().view(np.uint16), out["scattered_coord"].view(np.uint16))
    back = torch.empty_like(c4)
    pshattn.gather_rows(g, i2o, back)
    assert torch.equal(back, c4)


def test_scatter_index_empty_scenes(cuda_device):
    pts = np.concatenate([np.random.default_rng(0).uniform(-5, 5, (700, 3)), np.zeros((1, 3)),
                          np.full((900, 3), 1.25)]).astype(np.float32)
    seps = np.array([700, 700, 701, 1601])
    c16 = pts.astype(np.float16)
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 128, 1, 1700)
    ref_o2i, ref_i2o = po.scatter_index(out["bucket_id"], out["bucket_offs"], out["bucket_cumsum"], seps, 1700)
    o2i, i2o = _gpu_index(cuda_device, out, seps, 1700)
    assert np.array_equal(o2i.cpu().numpy(), ref_o2i) and np.array_equal(i2o.cpu().numpy(), ref_i2o)


@pytest.mark.parametrize("dtype,width", [(torch.bfloat16, 32), (torch.bfloat16, 36), (torch.float32, 3), (torch.float16, 6),
                                          (torch.uint8, 20), (torch.bfloat16, 512)])
def test_gather_rows_bit_exact(cuda_device, dtype, width):
    from flash3dtransformer_b200.lib import pshattn
    g = torch.Generator(device="cpu").manual_seed(width)
    rows_src, rows_out = 5003, 7001
    src = torch.randint(0, 255, (rows_src, width * torch.empty(0, dtype=dtype).element_size()), dtype=torch.uint8,
                        generator=g).view(dtype).to(cuda_device)
    index = torch.randint(0, rows_src + 40, (rows_out,), generator=g).to(torch.uint32)     # some past the end: zero rows
    out = torch.empty(rows_out, width, dtype=dtype, device=cuda_device)
    pshattn.gather_rows(src, index.to(cuda_device), out)
    ref = po.gather_rows(src.cpu().view(torch.uint8).numpy(), index.numpy())
    assert np.array_equal(out.cpu().view(torch.uint8).numpy(), ref)


def test_gather_rows_argument_errors(cuda_device):
    from flash3dtransformer_b200.lib import pshattn
    src = torch.zeros(10, 3, dtype=torch.bfloat16, device=cuda_device)                      # 6-byte rows
    idx = torch.zeros(4, dtype=torch.uint32, device=cuda_device)
    with pytest.raises(RuntimeError):
        pshattn.gather_rows(src, idx, torch.empty(4, 3, dtype=torch.bfloat16, device=cuda_device))
    ok = torch.zeros(10, 4, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(RuntimeError):
        pshattn.gather_rows(ok, idx, torch.empty(5, 4, dtype=torch.bfloat16, device=cuda_device))
    pshattn.gather_rows(ok, idx[:0], torch.empty(0, 4, dtype=torch.bfloat16, device=cuda_device))   # empty: no launch


@pytest.mark.parametrize("hash_type", [1, 2, 3, 4])
def test_kernel_output_against_the_reference_compiled_for_the_host(cuda_device, hash_type):
    """The kernels' bucketing goes through the reference's own scoreboard check (src/psh/bucket_sanitizer_cpu.cpp,
    compiled into oracle/_ref by oracle/ref_build.py), and every point that was not rebalanced carries the bucket id the
    reference's own hash lines (src/psh/hash_fns.cuh, same build) give it."""
    from oracle import ref_build
    import os
    san = ref_build.load_sanitizer()
    if san is None or not os.path.exists(ref_build.HASH_LIB):
        pytest.skip("oracle/_ref has not been built")
    sizes = [30000, 17001, 25013]
    coords32, seps = synthetic.batch(synthetic.lidar_scan, sizes, seed=6)
    c16 = coords32.astype(np.float16)
    nb, div, out = _gpu_scatter(cuda_device, c16, seps, 256, hash_type, c16.shape[0])
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).view(dt)
    cnt = t(out["bucket_cntr"], torch.uint32)
    maxcnt = torch.max(cnt.to(torch.int32), dim=-1)[0].to(torch.uint32)
    table = torch.zeros((len(sizes), nb, int(torch.max(cnt.to(torch.int32)))), dtype=torch.int8)
    res = cnt.clone()
    san.batch_bucket_sanitizer_cpu(t(out["bucket_id"], torch.uint16), cnt, t(out["bucket_offs"], torch.uint32), table, res,
                                   t(seps.astype(np.uint32), torch.uint32), maxcnt, len(sizes), nb)
    assert int(res.to(torch.int64).sum()) == 0
    _, h = ref_build.RefHash().vox_hash(c16, c16.min(0), c16.max(0), 0xFFFF, div, nb)
    first = h[hash_type - 1]
    kept = out["bucket_id"] == first
    # points leave their first bucket only when it overflowed (src/psh/batch_psh_bucket.cuh:157-246)
    assert kept.mean() > 0.5
    start = 0
    for s, end in enumerate(seps):
        ids, f = out["bucket_id"][start:end], first[start:end]
        full = np.bincount(f, minlength=nb) > 256
        assert np.all(full[f[ids != f]] | (f[ids != f] == 0))
        start = end


def test_flat_axis_bit_exact(cuda_device):
    # every point at the same height: the voxel quotient of that axis is 0/0 (the reference's clamp keeps the top voxel)
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [9000, 7000], seed=2)
    coords32[:, 2] = -1.5
    c16 = coords32.astype(np.float16)
    for hash_type in (1, 2):
        nb, div, out = _gpu_scatter(cuda_device, c16, seps, 256, hash_type, c16.shape[0])
        _compare(out, _oracle(c16, seps, nb, div, 256, hash_type, c16.shape[0]))
