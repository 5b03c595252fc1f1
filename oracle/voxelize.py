"""TEST INFRASTRUCTURE (not part of the product): CPU restatement of the
reference's point-to-voxel algorithm, PointToVoxel.generate_voxel_with_id,
spconv_triton/pytorch/utils.py:72-163, in numpy.  Pinned by
tests/test_oracle_golden.py against the reference's own frozen vectors
(tests/data/golden_ext_p2v.pt, CPU cases, bitwise) and against vectors made by
running the reference class here (tests/golden/make_golden.py)."""

from __future__ import annotations

import numpy as np


def point_to_voxel(points, vsize_xyz, coors_range_xyz, num_point_features, max_num_voxels,
                   max_num_points_per_voxel, empty_mean=False):
    """``(voxels [M, P, F] f32, indices [M, ndim] i32 zyx, num_per_voxel [M] i32,
    pc_voxel_id [N] i64)`` for float32 ``points`` [N, >= ndim]."""
    pc = np.asarray(points, dtype=np.float32)
    ndim = len(vsize_xyz)
    n = pc.shape[0]
    cmin = np.asarray(coors_range_xyz[:ndim], dtype=np.float32)
    cmax = coors_range_xyz[ndim:]
    vsize = np.asarray(vsize_xyz, dtype=np.float32)
    grid = [round((cmax[i] - coors_range_xyz[i]) / vsize_xyz[i]) for i in range(ndim)]  # utils.py:38-40
    pc_voxel_id = np.full(n, -1, dtype=np.int64)
    maxpts = max_num_points_per_voxel
    empty = (np.zeros((0, maxpts, num_point_features), np.float32), np.zeros((0, ndim), np.int32),
             np.zeros((0,), np.int32), pc_voxel_id)
    if n == 0:
        return empty
    with np.errstate(invalid="ignore", divide="ignore"):
        q = np.floor((pc[:, :ndim] - cmin) / vsize)  # utils.py:90, in float32
    in_range = np.all((q >= 0) & (q < np.asarray(grid, dtype=np.float32)), axis=1)  # NaN fails both
    valid_idx = np.nonzero(in_range)[0]
    if valid_idx.size == 0:
        return empty
    qv = q[valid_idx].astype(np.int64)
    lin = qv[:, 0]
    for d in range(1, ndim):
        lin = lin * int(grid[d]) + qv[:, d]  # utils.py:105-107
    uniq, first_pos, inverse = np.unique(lin, return_index=True, return_inverse=True)
    first_seen = valid_idx[first_pos]  # lowest point index of each voxel (utils.py:110-114)
    voxel_order = np.argsort(first_seen, kind="stable")
    vid_of_uniq = np.empty_like(voxel_order)
    vid_of_uniq[voxel_order] = np.arange(uniq.size)
    vid = vid_of_uniq[inverse]
    num_voxels = min(int(uniq.size), max_num_voxels)
    kept = vid < num_voxels
    counts = np.bincount(vid[kept], minlength=num_voxels)
    num_per_voxel = np.minimum(counts, maxpts).astype(np.int32)  # utils.py:119-120
    rem = uniq[voxel_order][:num_voxels]
    coords = np.empty((num_voxels, ndim), dtype=np.int64)
    for d in range(ndim - 1, -1, -1):
        coords[:, d] = rem % int(grid[d])
        rem = rem // int(grid[d])
    indices = coords[:, ::-1].astype(np.int32)  # z, y, x (utils.py:122-128)
    voxels = np.zeros((num_voxels, maxpts, num_point_features), dtype=np.float32)
    slot_of = np.zeros(num_voxels, dtype=np.int64)
    for i, v in zip(valid_idx[kept], vid[kept]):  # arrival order (utils.py:130-144)
        s = slot_of[v]
        if s < maxpts:
            voxels[v, s] = pc[i, :num_point_features]
        slot_of[v] = s + 1
    pc_voxel_id[valid_idx[kept]] = vid[kept]
    if empty_mean:  # utils.py:146-153
        for v in range(num_voxels):
            npv = int(num_per_voxel[v])
            s = np.zeros(num_point_features, dtype=np.float32)
            for k in range(maxpts):
                s = s + voxels[v, k]
            voxels[v, npv:] = s / np.float32(max(npv, 1))
    return voxels, indices, num_per_voxel, pc_voxel_id
