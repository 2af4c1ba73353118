"""Pins of the oracle and of the scoreboard operator on the REFERENCE's own code.

  * tests/golden/ref_hash.npz holds outputs of the reference's vox_coord and its four first-level hashes
    (src/psh/hash_fns.cuh:23-33,48-68,79-86,113-135), produced by oracle/ref_build.py from the reference's header
    compiled for the host; oracle/psh_oracle.py must reproduce every value.  Runs everywhere.
  * Where oracle/_ref/ has been built (or a reference checkout is present to build it from), the same comparison runs
    live on a million random points plus every boundary voxel, and the reference's bucket_sanitizer_cpu.cpp
    (src/psh/bucket_sanitizer_cpu.cpp:92-176) is run side by side with the library's f3d_batch_bucket_sanitizer_cpu
    and the oracle's scoreboard_check.
The reference's GPU binaries are built with --use_fast_math (CMakeLists.txt:50): their approximate division can move a
point that lies within rounding of a voxel boundary into the neighbouring voxel.  The host build divides exactly, and
so do this repository's kernels; `test_fast_math_exposure` counts how many points of a scan are that close.
"""
import os

import numpy as np
import pytest
import torch

from flash3dtransformer_b200 import synthetic
from flash3dtransformer_b200.lib import pshattn
from oracle import psh_oracle as po
from oracle import ref_build

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _check(vox_ref, hash_ref, vox, divisor, nb):
    assert np.array_equal(vox_ref.astype(np.uint32), vox)
    for t in (1, 2, 3, 4):
        assert np.array_equal(hash_ref[t - 1].astype(np.uint32), po.first_hash(t, vox, divisor, nb)), t


def test_oracle_reproduces_the_reference_hash_vectors():
    z = np.load(os.path.join(G, "ref_hash.npz"))
    pts, flat, vox = z["pts"], z["flat"], z["vox"]
    for nb in (128, 512, 2048):
        div = -(-0xFFFF // nb)
        _check(z["pts_vox"], z[f"pts_hash_{nb}"], po.vox_coords(pts, pts.min(0), pts.max(0), 0xFFFF), div, nb)
        _check(z["flat_vox"], z[f"flat_hash_{nb}"], po.vox_coords(flat, flat.min(0), flat.max(0), 0xFFFF), div, nb)
        v = vox.astype(np.uint32)
        for t in (1, 2, 3, 4):
            assert np.array_equal(z[f"vox_hash_{nb}"][t - 1].astype(np.uint32), po.first_hash(t, v, div, nb)), (nb, t)
    assert np.all(z["flat_vox"][:, 2] == 0xFFFE)          # the flat axis: 0/0 -> top voxel
    # the committed inputs are the ones the generator makes
    gp, gf, gv = ref_build.golden_inputs()
    assert np.array_equal(gp.view(np.uint16), pts.view(np.uint16)) and np.array_equal(gv, vox)


@pytest.fixture(scope="module")
def ref_hash():
    if not os.path.exists(ref_build.HASH_LIB):
        if not ref_build.have_reference():
            pytest.skip("oracle/_ref is not built and no reference checkout is present")
        ref_build.build_hash()
    return ref_build.RefHash()


def test_live_million_points_and_all_boundary_voxels(ref_hash):
    rng = np.random.default_rng(7)
    # LiDAR-like and box-like clouds, a million points together
    c32, _ = synthetic.batch(synthetic.lidar_scan, [500000], seed=11)
    box = rng.random((500000, 3), dtype=np.float32) * np.float32([100, 100, 8])
    for pts32 in (c32, box):
        pts = pts32.astype(np.float16)
        lo, hi = pts.min(0), pts.max(0)
        for nb in (64, 256, 2048):
            div = -(-0xFFFF // nb)
            v, h = ref_hash.vox_hash(pts, lo, hi, 0xFFFF, div, nb)
            _check(v, h, po.vox_coords(pts, lo, hi, 0xFFFF), div, nb)
    # every representable fp16 value of an axis (all voxel boundaries of that axis are crossed)
    axis = np.arange(0x0000, 0x7C00, dtype=np.uint16).view(np.float16)            # all finite non-negative halves
    pts = np.stack([axis, axis[::-1], -axis], axis=1)
    lo, hi = pts.min(0), pts.max(0)
    v, h = ref_hash.vox_hash(pts, lo, hi, 0xFFFF, 512, 128)
    _check(v, h, po.vox_coords(pts, lo, hi, 0xFFFF), 512, 128)
    # all 65536 voxel values on each axis in turn, the other two random
    allv = np.arange(65536, dtype=np.uint16)
    for axis_i in range(3):
        vox = rng.integers(0, 65536, (65536, 3)).astype(np.uint16)
        vox[:, axis_i] = allv
        for nb in (128, 1024):
            div = -(-0xFFFF // nb)
            h = ref_hash.hash_of_vox(vox, div, nb)
            for t in (1, 2, 3, 4):
                assert np.array_equal(h[t - 1].astype(np.uint32), po.first_hash(t, vox.astype(np.uint32), div, nb))


def test_fast_math_exposure():
    """How close points of a scan come to a voxel boundary: the quotient's distance to the next integer in units of its
    own rounding step.  Only points within a few steps could change voxel under an approximate division."""
    c32, _ = synthetic.batch(synthetic.lidar_scan, [120000], seed=0)
    c = c32.astype(np.float16).astype(np.float32)
    lo, hi = c.min(0), c.max(0)
    t = ((c - lo) * np.float32(0xFFFF)) / (hi - lo)
    frac = t - np.floor(t)
    ulp = np.spacing(np.maximum(t, np.float32(1)))
    near = np.minimum(frac, 1 - frac) <= 2 * ulp
    # points exactly on a boundary (fp16 grid values) are the exposed ones; they are a small share of a scan
    assert near.mean() < 0.05


@pytest.fixture(scope="module")
def ref_sanitizer():
    mod = ref_build.load_sanitizer()
    if mod is None:
        if not ref_build.have_reference():
            pytest.skip("oracle/_ref is not built and no reference checkout is present")
        mod = ref_build.build_sanitizer()
    return mod


def _bucketing(hash_type):
    c32, seps = synthetic.batch(synthetic.lidar_scan, [5000, 3100, 4200], seed=9)
    c16 = c32.astype(np.float16)
    nb, div = po.psh_params([5000, 3100, 4200], 128)
    out = po.psh_scatter(c16, seps, nb, div, 128, 0xFFFF, c16.min(0), c16.max(0), po.probe_table(), len(c16), 0.0, hash_type)
    as_t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).view(dt)
    return (as_t(out["bucket_id"].astype(np.uint16), torch.uint16), as_t(out["bucket_cntr"].astype(np.uint32), torch.uint32),
            as_t(out["bucket_offs"].astype(np.uint32), torch.uint32), as_t(seps.astype(np.uint32), torch.uint32), nb, out, seps)


def _args(bid, cnt, off, sp, nb):
    maxcnt = torch.max(cnt.to(torch.int32), dim=-1)[0].to(torch.uint32)
    table = torch.zeros((sp.numel(), nb, int(torch.max(cnt.to(torch.int32)))), dtype=torch.int8)
    return [bid, cnt, off, table, cnt.clone(), sp, maxcnt, sp.numel(), nb]


@pytest.mark.parametrize("hash_type", [1, 2, 3, 4])
def test_scoreboard_operator_agrees_with_the_reference_source(ref_sanitizer, hash_type):
    bid, cnt, off, sp, nb, out, seps = _bucketing(hash_type)
    a, b = _args(bid, cnt, off, sp, nb), _args(bid, cnt, off, sp, nb)
    ref_sanitizer.batch_bucket_sanitizer_cpu(*a)             # the reference's code accepts the oracle's bucketing ...
    pshattn.batch_bucket_sanitizer_cpu(*b)                   # ... and so does the library's operator,
    assert torch.equal(a[3], b[3]) and torch.equal(a[4].view(torch.int32), b[4].view(torch.int32))   # same in/out
    po.scoreboard_check(out["bucket_id"], out["bucket_cntr"], out["bucket_offs"], seps, nb)
    # violations: both raise, on the same kind of message
    def poke(t, i, v):
        w = t.view(torch.int16 if t.dtype == torch.uint16 else torch.int32).clone()
        w[i] = v
        return w.view(t.dtype)
    same_bucket = (bid.view(torch.int16)[:5000] == bid.view(torch.int16)[0]).nonzero()
    cases = {"Wrong scoreboard": (bid, poke(off, int(same_bucket[1]), int(off.view(torch.int32)[0]))),
             "overflow": (poke(bid, 7, nb + 1), off)}
    for msg, (bid2, off2) in cases.items():
        for fn in (ref_sanitizer.batch_bucket_sanitizer_cpu, pshattn.batch_bucket_sanitizer_cpu):
            with pytest.raises(RuntimeError, match=msg):
                fn(*_args(bid2, cnt, off2, sp, nb))
