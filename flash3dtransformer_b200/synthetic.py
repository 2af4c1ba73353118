"""Seeded synthetic point clouds with the shapes, sizes and value distributions of the benchmark configurations.

The reference measures on KITTI velodyne scans read from $KITTI_RT (tests/test_psh.py:25-44); that dataset is
not available here, so these generators stand in for it.  All return fp32 xyz as numpy arrays; callers cast to
fp16 for the operators, as the reference's tests do (tests/test_psh.py:43).
"""
from __future__ import annotations

import numpy as np


def ground_and_blobs(n: int = 20000, seed: int = 0) -> np.ndarray:
    """70 % of the points on a ground slab z in [-2,-1.8] m over x,y in [-25,25] m, 30 % on 20 Gaussian blobs
    (sigma 0.5 m) with centres uniform in x,y in [-25,25] m, z in [-2,2] m."""
    rng = np.random.default_rng(seed)
    n_ground = int(round(0.7 * n))
    n_blob = n - n_ground
    ground = np.stack([rng.uniform(-25, 25, n_ground), rng.uniform(-25, 25, n_ground),
                       rng.uniform(-2.0, -1.8, n_ground)], axis=1)
    centres = np.stack([rng.uniform(-25, 25, 20), rng.uniform(-25, 25, 20), rng.uniform(-2, 2, 20)], axis=1)
    which = np.arange(n_blob) % 20
    blobs = centres[which] + rng.normal(0.0, 0.5, (n_blob, 3))
    pts = np.concatenate([ground, blobs], axis=0).astype(np.float32)
    return pts[rng.permutation(n)]


def lidar_scan(n: int = 120000, seed: int = 0) -> np.ndarray:
    """LiDAR-like scan: 64 elevation rings over [-25 deg, 3 deg], uniform azimuth, range with density ~ 1/r on
    [2, 80] m (r = 2 * 40**u, u uniform).  Points are ordered ring by ring along the azimuth, the order in which a
    spinning sensor delivers them."""
    rng = np.random.default_rng(seed)
    elev = np.deg2rad(np.linspace(-25.0, 3.0, 64))
    ring = rng.integers(0, 64, n)
    az = rng.uniform(0.0, 2.0 * np.pi, n)
    r = 2.0 * np.power(40.0, rng.uniform(0.0, 1.0, n))
    e = elev[ring]
    pts = np.stack([r * np.cos(e) * np.cos(az), r * np.cos(e) * np.sin(az), r * np.sin(e)], axis=1)
    order = np.lexsort((az, ring))
    return pts[order].astype(np.float32)


def zipf_voxels(n: int = 1_000_000, seed: int = 0, voxel: float = 0.05, alpha: float = 1.5,
                box=(100.0, 100.0, 8.0)) -> np.ndarray:
    """Heavy-tailed occupancy: occupied voxels uniform in the box, points per voxel ~ Zipf(alpha) truncated so the
    total is exactly n, points uniform inside their voxel."""
    rng = np.random.default_rng(seed)
    counts = []
    total = 0
    while total < n:
        c = rng.zipf(alpha, size=max(1024, n // 8)).astype(np.int64)
        c = np.minimum(c, n)
        counts.append(c)
        total += int(c.sum())
    counts = np.concatenate(counts)
    csum = np.cumsum(counts)
    last = int(np.searchsorted(csum, n))
    counts = counts[: last + 1].copy()
    counts[last] -= int(csum[last] - n)
    counts = counts[counts > 0]
    nvox = counts.shape[0]
    dims = np.asarray(box) / voxel
    vox = np.stack([rng.integers(0, int(dims[d]), nvox) for d in range(3)], axis=1).astype(np.float64)
    owner = np.repeat(np.arange(nvox), counts)
    pts = (vox[owner] + rng.uniform(0.0, 1.0, (owner.shape[0], 3))) * voxel
    pts -= np.asarray(box) / 2.0
    return pts.astype(np.float32)


def batch(scene_fn, sizes, seed: int = 0):
    """Concatenate scenes; returns (coords fp32 [N,3], seps int64 [B] = inclusive end rows)."""
    scenes = [scene_fn(int(n), seed + i) for i, n in enumerate(sizes)]
    coords = np.concatenate(scenes, axis=0) if scenes else np.zeros((0, 3), np.float32)
    seps = np.cumsum(np.asarray([s.shape[0] for s in scenes], dtype=np.int64))
    return coords, seps
