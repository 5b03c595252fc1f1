"""Point-to-voxel on the GPU through the C ABI: bitwise against the reference's
frozen CPU vectors and the vectors made by the reference class, against the
oracle on a LiDAR-sized cloud, and the structural checks of the reference's
tests/test_ext_p2v.py:52-93."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle.voxelize import point_to_voxel
from test_oracle_voxelize import FROZEN_CANON, FROZEN_CPU, GOLD, canon

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda")


def P2V(**ctor):
    from spconv_triton_b200.pytorch.utils import PointToVoxel

    return PointToVoxel(device=DEV, **ctor)


def check(out, expect, mean_tol=0.0):
    vox, idx, npv, pcvid = (t.cpu().numpy() for t in out)
    np.testing.assert_array_equal(idx, np.asarray(expect["indices"]))
    np.testing.assert_array_equal(npv, np.asarray(expect["num_per_voxel"]))
    np.testing.assert_array_equal(pcvid, np.asarray(expect["pc_voxel_id"]))
    if mean_tol:
        np.testing.assert_allclose(vox, np.asarray(expect["voxels"]), rtol=0, atol=mean_tol)
    else:
        np.testing.assert_array_equal(vox, np.asarray(expect["voxels"]))


@pytest.mark.parametrize("case", FROZEN_CPU, ids=lambda c: c["id"])
def test_frozen_cpu_cases_bitwise(case):
    out = P2V(**case["ctor"]).generate_voxel_with_id(case["points"].to(DEV))
    check(out, case["expect"])


@pytest.mark.parametrize("case", FROZEN_CANON, ids=lambda c: c["id"])
def test_frozen_canonical_cases(case):
    vox, idx, npv, _ = P2V(**case["ctor"]).generate_voxel_with_id(case["points"].to(DEV))
    i, v, n = canon(idx.cpu().numpy(), vox.cpu().numpy(), npv.cpu().numpy())
    e = case["expect"]
    np.testing.assert_array_equal(i, e["indices_canon"].numpy())
    np.testing.assert_array_equal(n, e["num_per_voxel_canon"].numpy())
    if e["check_contents"]:
        np.testing.assert_allclose(v, e["voxels_canon"].numpy(), rtol=0, atol=1e-5)


@pytest.mark.parametrize("case", GOLD["generated"], ids=lambda c: c["id"])
def test_generated_cases(case):
    """Every call of the sequence, on one object: persistent buffers, clear_voxels
    off and empty_mean behave as the reference class does."""
    p2v = P2V(**case["ctor"])
    pts = case["points"].to(DEV)
    for (clear, mean), expect in zip(case["calls"], case["expect"]):
        out = p2v.generate_voxel_with_id(pts, clear_voxels=clear, empty_mean=mean)
        check(out, expect, mean_tol=1e-6 if mean else 0.0)


def test_lidar_sized_cloud_matches_oracle():
    g = torch.Generator().manual_seed(9)
    n = 300_000
    pts = torch.cat([torch.randn(n, 3, generator=g) * torch.tensor([25.0, 25.0, 1.2]), torch.rand(n, 2, generator=g)], 1)
    ctor = dict(vsize_xyz=[0.1, 0.1, 0.2], coors_range_xyz=[-51.2, -51.2, -5.0, 51.2, 51.2, 3.0],
                num_point_features=5, max_num_voxels=120_000, max_num_points_per_voxel=5)
    out = P2V(**ctor).generate_voxel_with_id(pts.to(DEV))
    exp = point_to_voxel(pts.numpy(), **ctor)
    check(out, dict(voxels=exp[0], indices=exp[1], num_per_voxel=exp[2], pc_voxel_id=exp[3]))
    assert out[1].shape[0] == 120_000  # the cap is reached: later voxels are dropped, their points get -1
    assert int((out[3] < 0).sum()) > 0


def test_cap_structural():
    g = torch.Generator().manual_seed(3)
    pc = torch.rand(500, 3, generator=g).to(DEV)
    cap = 20
    vox, idx, npv, pcvid = P2V(vsize_xyz=[0.05] * 3, coors_range_xyz=[0, 0, 0, 1, 1, 1], num_point_features=3,
                               max_num_voxels=cap, max_num_points_per_voxel=4).generate_voxel_with_id(pc)
    assert idx.shape[0] == cap
    assert int(pcvid.max()) == cap - 1
    assert int((pcvid < 0).sum()) > 0
    valid = pcvid >= 0
    q = (pc[valid] / 0.05).floor().long().flip(1)
    assert torch.equal(idx.long()[pcvid[valid]], q)


def test_truncation_keeps_voxel_id():
    pc = torch.tensor([[0.05, 0.05, 0.05], [0.051, 0.05, 0.05], [0.052, 0.05, 0.05], [0.3, 0.3, 0.3]], device=DEV)
    vox, idx, npv, pcvid = P2V(vsize_xyz=[0.1] * 3, coors_range_xyz=[0, 0, 0, 1, 1, 1], num_point_features=3,
                               max_num_voxels=10, max_num_points_per_voxel=2).generate_voxel_with_id(pc)
    assert pcvid.tolist() == [0, 0, 0, 1]
    assert npv.tolist() == [2, 1]
    assert idx.tolist() == [[0, 0, 0], [3, 3, 3]]
    assert torch.equal(vox[0], pc[:2])


def test_empty_and_wrong_inputs():
    from spconv_triton_b200.pytorch.utils import PointToVoxel, gather_features_by_pc_voxel_id
    from spconv_triton_b200.utils import Point2VoxelCPU3d, Point2VoxelGPU3d

    p2v = Point2VoxelGPU3d([0.1] * 3, [0, 0, 0, 1, 1, 1], 3, 10, 2)
    vox, idx, npv, pcvid = p2v.generate_voxel_with_id(torch.zeros(0, 3, device=DEV))
    assert vox.shape == (0, 2, 3) and idx.shape == (0, 3) and npv.shape == (0,) and pcvid.shape == (0,)
    with pytest.raises(AssertionError):
        p2v.generate_voxel_with_id(torch.zeros(4, 3))  # CPU points on a CUDA voxeliser
    with pytest.raises(NotImplementedError):
        Point2VoxelCPU3d([0.1] * 3, [0, 0, 0, 1, 1, 1], 3, 10, 2)  # no CPU path
    with pytest.raises(NotImplementedError):
        PointToVoxel([0.1] * 3, [0, 0, 0, 1, 1, 1], 3, 10, 2, DEV).generate_voxel_with_id(
            torch.zeros(4, 3, device=DEV, dtype=torch.float64))
    feats = torch.arange(6.0, device=DEV).view(3, 2)
    back = gather_features_by_pc_voxel_id(feats, torch.tensor([2, -1, 0], device=DEV), invalid_value=-7)
    assert back.tolist() == [[4.0, 5.0], [-7.0, -7.0], [0.0, 1.0]]
