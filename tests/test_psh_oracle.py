"""CPU tests of the PSH oracle: known answers of the published Philox algorithm, the reference's invariants
(tests/test_psh.py:117-129) on synthetic scans for all four hashes, and edge cases."""
import numpy as np
import pytest

from oracle import psh_oracle as po
from flash3dtransformer_b200 import synthetic


def test_philox_known_answers():
    # Known-answer vectors published with the Philox4x32-10 generator (Random123 kat_vectors)
    z = np.zeros(1, dtype=np.uint32)
    out = po.philox4x32_10(z, z, z, z, 0, 0)
    assert [int(x[0]) for x in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = np.full(1, 0xFFFFFFFF, dtype=np.uint32)
    out = po.philox4x32_10(f, f, f, f, 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(x[0]) for x in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]


def test_zorder_bit_selection():
    # (morton >> 31) & 0xFFFF keeps x[11..15], y[10..15], z[10..14]
    rng = np.random.default_rng(1)
    v = rng.integers(0, 65536, (4096, 3)).astype(np.uint32)
    h = po.zorder16(v[:, 0], v[:, 1], v[:, 2])
    exp = np.zeros(4096, dtype=np.uint32)
    for k in range(16):
        m = 31 + k
        src = v[:, m % 3]
        exp |= ((src >> np.uint32(m // 3)) & np.uint32(1)) << np.uint32(k)
    assert np.array_equal(h, exp)
    lowbits = v.copy()
    lowbits[:, 0] &= 0x07FF; lowbits[:, 1] &= 0x03FF; lowbits[:, 2] &= 0x83FF
    assert np.all(po.zorder16(lowbits[:, 0], lowbits[:, 1], lowbits[:, 2]) == 0)


def test_vox_clamp_and_degenerate_bbox():
    c = np.array([[0, 0, 0], [1, 1, 1], [2, 2, 2]], dtype=np.float16)
    v = po.vox_coords(c, c.min(0), c.max(0), 0xFFFF)
    assert v.min() == 0 and v.max() == 0xFFFE and np.all(v[1] == 32767)
    flat = np.array([[1, 2, 3], [1, 5, 3]], dtype=np.float16)
    v = po.vox_coords(flat, flat.min(0), flat.max(0), 0xFFFF)
    # a flat axis divides 0 by 0; the device's min / max drop the NaN, which leaves the top voxel (the reference's
    # own clamp compiled for the host gives the same: tests/test_ref_pins.py)
    assert np.all(v[:, 0] == 0xFFFE) and np.all(v[:, 2] == 0xFFFE) and v[0, 1] == 0 and v[1, 1] == 0xFFFE


def _run(coords32, seps, bucket_size, hash_type, pad_align=None):
    coords = coords32.astype(np.float16)
    sizes = np.diff(np.concatenate([[0], seps]))
    nb, div = po.psh_params(sizes, bucket_size)
    n = coords.shape[0]
    pad_to = n if pad_align is None else -(-n // pad_align) * pad_align
    out = po.psh_scatter(coords, seps, nb, div, bucket_size, 0xFFFF, coords.min(0), coords.max(0),
                         po.probe_table(), pad_to, 0.0, hash_type)
    return coords, nb, out


@pytest.mark.parametrize("hash_type", [1, 2, 3, 4])
def test_invariants_lidar(hash_type):
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [6000, 4500, 7000], seed=3)
    coords, nb, out = _run(coords32, seps, 256, hash_type, pad_align=256 * 6)
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)
    assert not np.isnan(out["scattered_coord"].astype(np.float32)).any()
    assert np.array_equal(np.cumsum(out["bucket_cntr"].astype(np.int64), 1), out["bucket_cumsum"].astype(np.int64))
    # the scatter is a permutation of every scene followed by zero padding
    start = 0
    for s in range(len(seps)):
        end = int(seps[s])
        a = np.sort(coords[start:end].view(np.uint16).astype(np.int64) @ np.array([1, 1 << 16, 1 << 32]))
        b = np.sort(out["scattered_coord"][start:end].view(np.uint16).astype(np.int64) @ np.array([1, 1 << 16, 1 << 32]))
        assert np.array_equal(a, b)
        assert out["bucket_cntr"][s].sum() == end - start
        start = end
    assert np.all(out["scattered_coord"][start:] == 0)
    # recycle bucket holds at most bucket_size once the redistribution has run
    assert np.all(out["bucket_cntr"][:, 0] <= 256)


def test_non_overflowing_points_keep_first_hash():
    coords32, seps = synthetic.batch(synthetic.ground_and_blobs, [20000], seed=0)
    coords, nb, out = _run(coords32, seps, 256, 2)
    assert nb == 128
    vox = po.vox_coords(coords, coords.min(0), coords.max(0), 0xFFFF)
    b0 = po.first_hash(2, vox, 512, nb)
    rank, _ = po.stable_rank(b0.astype(np.int64), nb)
    keep = (b0 == 0) | (rank < 256)
    moved_from_recycle = (b0 == 0) & (rank >= 256)
    stay = keep & ~moved_from_recycle
    assert np.array_equal(out["bucket_id"][stay], b0[stay].astype(np.uint16))
    assert np.array_equal(out["bucket_offs"][stay], rank[stay].astype(np.uint32))


def test_edge_cases():
    # empty scene in the middle, a single-point scene, every point in one voxel
    pts = np.concatenate([np.random.default_rng(0).uniform(-5, 5, (700, 3)), np.zeros((1, 3)),
                          np.full((900, 3), 1.25)]).astype(np.float32)
    seps = np.array([700, 700, 701, 1601])
    coords, nb, out = _run(pts, seps, 128, 1)
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)
    assert out["bucket_cntr"][1].sum() == 0 and out["bucket_cntr"][2].sum() == 1
    # all-identical scene: one bucket overflows massively, everything is still placed exactly once
    assert out["bucket_cntr"][3].sum() == 900
    with pytest.raises(ValueError):
        po.psh_scatter(coords, seps, nb, 1, 128, 0xFFFF, coords.min(0), coords.max(0), po.probe_table(),
                       coords.shape[0], 0.0, 1)
    with pytest.raises(ValueError):
        po.psh_scatter(coords, seps, nb, 65535, 128, 0xFFFF, coords.min(0), coords.max(0), po.probe_table(),
                       10, 0.0, 1)


def test_scatter_index_is_the_permutation_of_the_coordinate_scatter():
    # empty scene, single-point scene, odd sizes; padded past the input length
    coords32, seps = synthetic.batch(synthetic.lidar_scan, [3000, 1, 4500], seed=11)
    seps = np.array([seps[0], seps[0], seps[1], seps[2]])
    coords, nb, out = _run(coords32, seps, 128, 2, pad_align=128 * 6)
    n, pad_to = coords.shape[0], out["scattered_coord"].shape[0]
    out2in, in2out = po.scatter_index(out["bucket_id"], out["bucket_offs"], out["bucket_cumsum"], seps, pad_to)
    assert np.array_equal(out2in[in2out], np.arange(n))
    assert np.all(out2in[n:] == n + 3) and np.all(out2in[:n] < n)
    # gathering the input coordinates through out2in reproduces the scatter (padding rows are zero)
    assert np.array_equal(po.gather_rows(coords, out2in).view(np.uint16), out["scattered_coord"].view(np.uint16))
    # and in2out brings them back
    assert np.array_equal(po.gather_rows(out["scattered_coord"], in2out).view(np.uint16), coords.view(np.uint16))
    # a scene keeps its row range
    start = 0
    for end in seps:
        assert np.all((in2out[start:end] >= start) & (in2out[start:end] < end))
        start = end
