"""Seeded synthetic voxel scenes with the shapes and distributions of the
benchmark configurations (stand-ins for LiDAR / indoor-scan data sets; no data
set is read).  numpy only; used by bench.py and by the tests."""

from __future__ import annotations

import numpy as np


def _unique_rows(coords, shape):
    lin = np.ravel_multi_index(tuple(coords.T), shape)
    _, first = np.unique(lin, return_index=True)
    return coords[np.sort(first)]


def lidar_like_sample(rng, n_target, grid=(41, 1600, 1408), n_clusters=200, sigma=8.0, ground_frac=0.7):
    """(z, y, x) int32 [n_target, 3], unique: ``ground_frac`` of the voxels on a
    noisy ground plane z = clamp(round(2 + N(0,1)), 0, 4) with (y, x) uniform,
    the rest in ``n_clusters`` isotropic Gaussian clusters (sigma in voxels)
    around centres drawn uniformly in the grid, clamped to the grid."""
    grid = np.asarray(grid)
    out = np.zeros((0, 3), dtype=np.int64)
    centres = np.stack([rng.integers(0, g, n_clusters) for g in grid], 1)
    while out.shape[0] < n_target:
        need = n_target - out.shape[0]
        m = int(need * 1.3) + 64
        n_g = int(m * ground_frac)
        ground = np.stack([
            np.clip(np.rint(2 + rng.standard_normal(n_g)), 0, 4),
            rng.integers(0, grid[1], n_g),
            rng.integers(0, grid[2], n_g),
        ], 1).astype(np.int64)
        n_c = m - n_g
        which = rng.integers(0, n_clusters, n_c)
        cl = np.rint(centres[which] + rng.standard_normal((n_c, 3)) * sigma).astype(np.int64)
        cl = np.clip(cl, 0, grid - 1)
        new = np.concatenate([ground, cl], 0)
        new = new[rng.permutation(new.shape[0])]
        out = _unique_rows(np.concatenate([out, new], 0), tuple(grid))
    return out[:n_target].astype(np.int32)


def lidar_like_batch(seed, batch, n_range, grid=(41, 1600, 1408), **kw):
    """int32 indices [N, 4] (batch, z, y, x), rows grouped by sample; the
    per-sample voxel count is an integer drawn uniformly from ``n_range``."""
    rng = np.random.default_rng(seed)
    rows = []
    for b in range(batch):
        n = int(rng.integers(n_range[0], n_range[1] + 1))
        c = lidar_like_sample(rng, n, grid, **kw)
        rows.append(np.concatenate([np.full((n, 1), b, np.int32), c], 1))
    return np.concatenate(rows, 0)


def uniform_batch(seed, batch, n_per_sample, grid):
    """Unique coordinates drawn uniformly without replacement."""
    rng = np.random.default_rng(seed)
    rows = []
    vol = int(np.prod(grid))
    for b in range(batch):
        lin = rng.choice(vol, size=n_per_sample, replace=False)
        c = np.stack(np.unravel_index(lin, grid), 1).astype(np.int32)
        rows.append(np.concatenate([np.full((n_per_sample, 1), b, np.int32), c], 1))
    return np.concatenate(rows, 0)


def indoor_like_sample(rng, n_target, grid=(512, 512, 64)):
    """(x, y, z) int32 [n_target, 3], unique: the six walls of 3-6 random
    axis-aligned boxes plus 2-4 random tilted planes, rasterised to voxels and
    sub-sampled to ``n_target`` (fewer if the surfaces hold fewer voxels)."""
    gx, gy, gz = (int(g) for g in grid)
    parts = []
    for _ in range(int(rng.integers(3, 7))):
        lo = np.array([rng.integers(0, gx - 64), rng.integers(0, gy - 64), rng.integers(0, max(gz - 24, 1))])
        ext = np.array([rng.integers(48, 256), rng.integers(48, 256), rng.integers(12, max(gz // 2, 13))])
        hi = np.minimum(lo + ext, [gx - 1, gy - 1, gz - 1])
        xs, ys, zs = (np.arange(lo[d], hi[d] + 1) for d in range(3))
        for d, (a, b) in enumerate(((ys, zs), (xs, zs), (xs, ys))):
            u, v = np.meshgrid(a, b, indexing="ij")
            for face in (lo[d], hi[d]):
                cols = [None, None, None]
                cols[d] = np.full(u.size, face)
                others = [c for c in range(3) if c != d]
                cols[others[0]], cols[others[1]] = u.ravel(), v.ravel()
                parts.append(np.stack(cols, 1))
    xs, ys = np.meshgrid(np.arange(gx), np.arange(gy), indexing="ij")
    for _ in range(int(rng.integers(2, 5))):
        a, b = rng.uniform(-0.08, 0.08, 2)
        c = rng.uniform(0.2, 0.8) * gz
        z = np.rint(a * (xs - gx / 2) + b * (ys - gy / 2) + c).astype(np.int64)
        ok = (z >= 0) & (z < gz)
        parts.append(np.stack([xs[ok], ys[ok], z[ok]], 1))
    pts = _unique_rows(np.concatenate(parts, 0).astype(np.int64), (gx, gy, gz))
    pts = pts[rng.permutation(pts.shape[0])[:n_target]]
    return pts.astype(np.int32)


def indoor_like_batch(seed, batch, n_range, grid=(512, 512, 64)):
    """int32 indices [N, 4] (batch, x, y, z), rows grouped by sample; the
    per-sample voxel count is an integer drawn uniformly from ``n_range``."""
    rng = np.random.default_rng(seed)
    rows = []
    for b in range(batch):
        n = int(rng.integers(n_range[0], n_range[1] + 1))
        c = indoor_like_sample(rng, n, grid)
        rows.append(np.concatenate([np.full((c.shape[0], 1), b, np.int32), c], 1))
    return np.concatenate(rows, 0)


def blob_batch(seed, batch, n_per_sample, grid=256, occupancy=0.3):
    """int32 indices [batch * n_per_sample, 4] (batch, z, y, x): random solid blobs (spheres of radius
    grid/32 .. grid/10) are placed until they hold n_per_sample / occupancy cells, and
    ``n_per_sample`` of those cells are kept at random, so that the voxels fill their blobs to
    ``occupancy`` ("dense-ish ... 30 % occupancy in random blobs").  Rows of a sample are in random order."""
    rng = np.random.default_rng(seed)
    rows = []
    want = int(n_per_sample / occupancy)
    for b in range(batch):
        filled = np.zeros((grid, grid, grid), dtype=bool)
        count = 0
        while count < want:
            r = int(rng.integers(max(grid // 32, 3), max(grid // 10, 5)))
            c = rng.integers(r, grid - r, size=3)
            ax = np.arange(-r, r + 1)
            ball = (ax[:, None, None] ** 2 + ax[None, :, None] ** 2 + ax[None, None, :] ** 2) <= r * r
            view = filled[c[0] - r:c[0] + r + 1, c[1] - r:c[1] + r + 1, c[2] - r:c[2] + r + 1]
            count += int((ball & ~view).sum())
            view |= ball
        cells = np.flatnonzero(filled)
        keep = cells[rng.permutation(cells.shape[0])[:n_per_sample]]
        zyx = np.stack(np.unravel_index(keep, filled.shape), 1)
        rows.append(np.concatenate([np.full((zyx.shape[0], 1), b), zyx], 1))
    return np.concatenate(rows).astype(np.int32)
