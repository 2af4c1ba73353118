"""Scan-file front end: reading fp32 point records, and the device collate against the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from oracle import psh_oracle as po
from flash3dtransformer_b200 import synthetic


def _write_scans(tmp_path, sizes, dim, seed=0):
    rng = np.random.default_rng(seed)
    paths, recs = [], []
    for i, n in enumerate(sizes):
        xyz = synthetic.lidar_scan(n, seed + i) if n else np.zeros((0, 3), np.float32)
        rec = np.concatenate([xyz.astype(np.float32), rng.uniform(0, 1, (n, dim - 3)).astype(np.float32)], axis=1)
        p = tmp_path / f"scan_{i}.bin"
        rec.tofile(p)
        paths.append(str(p)); recs.append(rec)
    return paths, np.concatenate(recs, axis=0)


def test_read_scan_bins(tmp_path):
    from flash3dtransformer_b200.psh import scan_io
    paths, ref = _write_scans(tmp_path, [1000, 0, 37, 4096], 4)
    host, sizes = scan_io.read_scan_bins(paths, 4)
    assert sizes == [1000, 0, 37, 4096] and host.dtype == torch.float32
    assert np.array_equal(host.numpy(), ref)
    # five floats per point (ring index) and a truncated file
    paths5, ref5 = _write_scans(tmp_path, [33], 5, seed=3)
    host5, sizes5 = scan_io.read_scan_bins(paths5, 5)
    assert sizes5 == [33] and np.array_equal(host5.numpy(), ref5)
    with pytest.raises(ValueError):
        scan_io.read_scan_bins(paths5, 4)           # 33 * 20 bytes is not a multiple of 16
    with pytest.raises(ValueError):
        scan_io.read_scan_bins(paths, 2)


def test_oracle_collate_matches_host_collate():
    """The oracle's cast + slice equals collate_coords_flat_sep, whose outputs are pinned by the golden fixtures."""
    from flash3dtransformer_b200.psh import batching
    rng = np.random.default_rng(1)
    scenes = [rng.normal(0, 30, (n, 4)).astype(np.float32) for n in (100, 1, 257)]
    coords, seps = batching.collate_coords_flat_sep([torch.from_numpy(s) for s in scenes], torch.float16, torch.uint32)
    oc, extra, oseps = po.collate_points(np.concatenate(scenes), [100, 1, 257])
    assert np.array_equal(coords.numpy().view(np.uint16), oc.view(np.uint16))
    assert np.array_equal(seps.to(torch.int64).numpy(), oseps.astype(np.int64))
    assert extra.shape == (358, 1)


@pytest.mark.gpu
@pytest.mark.parametrize("dim,sizes", [(4, [120000, 1, 4097]), (4, [1024]), (4, [1023]), (5, [5000, 3000]), (3, [2049]), (6, [777])])
def test_collate_points_bit_exact(cuda_device, tmp_path, dim, sizes):
    from flash3dtransformer_b200.psh import scan_io
    paths, ref = _write_scans(tmp_path, sizes, dim, seed=dim)
    # values that exercise the conversion: halfway cases, overflow to inf, subnormal halves, negative zero
    special = np.array([2049.0, 2051.0, 65519.9, 65520.0, 1e-7, 6e-8, -0.0, 1.00048828125], dtype=np.float32)
    ref[: len(special), 0] = special
    ref[: len(special), 2] = -special
    off = 0
    for p, n in zip(paths, sizes):
        ref[off:off + n].tofile(p)
        off += n
    coords, extra, seps = scan_io.load_scans(paths, cuda_device, dim)
    torch.cuda.synchronize()
    oc, oe, oseps = po.collate_points(ref, sizes)
    assert np.array_equal(coords.cpu().numpy().view(np.uint16), oc.view(np.uint16))
    if dim > 3:
        assert np.array_equal(extra.cpu().numpy(), oe)
    else:
        assert extra is None
    assert np.array_equal(seps.cpu().to(torch.int64).numpy(), oseps.astype(np.int64))
    assert getattr(seps, "_f3d_host", None) is not None


@pytest.mark.gpu
def test_loaded_scans_run_through_the_psh_scatter(cuda_device, tmp_path):
    from flash3dtransformer_b200.psh import psh_main as pm, scan_io
    paths, ref = _write_scans(tmp_path, [30000, 22000], 4, seed=8)
    coords, extra, seps = scan_io.load_scans(paths, cuda_device, 4)
    pad_to = -(-coords.shape[0] // 512) * 512
    scattered, buffers = pm.batch_bucket_scatter(coords, seps, 512, pad_to, 2)
    out2in, in2out = pm.scatter_index(buffers, seps, pad_to)
    torch.cuda.synchronize()
    assert torch.equal(scattered[in2out.long()], coords)
    with pytest.raises(RuntimeError):
        scan_io.collate_scans(torch.zeros(10, 4), [4, 5], cuda_device)
