"""Generate tests/golden/ref_p2v.pt: golden vectors of the point-to-voxel step.

Run once where the reference checkout is readable at $SPCONV_REFERENCE_ROOT:

    python tests/golden/make_golden_p2v.py

Two kinds of cases are written:
1. ``frozen``: the cases of the reference's own tests/data/golden_ext_p2v.pt,
   re-saved unchanged (three CPU cases checked bitwise upstream, two canonical
   1-D / 4-D cases);
2. ``generated``: outputs of the reference's PointToVoxel class itself (pure
   torch, run here on the CPU) on seeded points: voxel cap, truncation,
   empty_mean, clear_voxels=False reuse, 1/2/4-D, points outside the range and
   on cell boundaries, NaN coordinates, more columns than stored features.

Nothing here is imported by the product or by the tests.
"""

import importlib.util
import os
from pathlib import Path

import torch

REF = Path(os.environ["SPCONV_REFERENCE_ROOT"])  # the read-only reference checkout
OUT = Path(__file__).parent / "ref_p2v.pt"

spec = importlib.util.spec_from_file_location("ref_p2v_utils", REF / "spconv_triton" / "pytorch" / "utils.py")
ref = importlib.util.module_from_spec(spec)
spec.loader.exec_module(ref)


def run(ctor, points, calls):
    """``calls``: list of (clear_voxels, empty_mean); the same object serves them in turn."""
    p2v = ref.PointToVoxel(device=torch.device("cpu"), **ctor)
    outs = []
    for clear, mean in calls:
        vox, idx, npv, pcvid = p2v.generate_voxel_with_id(points, clear_voxels=clear, empty_mean=mean)
        outs.append(dict(voxels=vox, indices=idx, num_per_voxel=npv, pc_voxel_id=pcvid))
    return outs


def main():
    frozen = torch.load(REF / "tests" / "data" / "golden_ext_p2v.pt", map_location="cpu", weights_only=False)["cases"]
    g = torch.Generator().manual_seed(20240607)
    cases = []

    def add(name, ctor, points, calls=((True, False),)):
        cases.append(dict(id=name, ctor=ctor, points=points, calls=list(calls), expect=run(ctor, points, calls)))

    lidar = torch.cat([torch.randn(6000, 3, generator=g) * torch.tensor([20.0, 20.0, 1.0]),
                       torch.rand(6000, 1, generator=g)], 1)
    add("lidar_like", dict(vsize_xyz=[0.5, 0.5, 0.25], coors_range_xyz=[-40, -40, -3, 40, 40, 1],
                           num_point_features=4, max_num_voxels=20000, max_num_points_per_voxel=5), lidar)
    add("lidar_cap_mean", dict(vsize_xyz=[1.0, 1.0, 0.5], coors_range_xyz=[-40, -40, -3, 40, 40, 1],
                               num_point_features=4, max_num_voxels=300, max_num_points_per_voxel=3), lidar,
        calls=((True, True),))
    add("reuse_no_clear", dict(vsize_xyz=[2.0, 2.0, 1.0], coors_range_xyz=[-40, -40, -3, 40, 40, 1],
                               num_point_features=3, max_num_voxels=5000, max_num_points_per_voxel=4), lidar,
        calls=((True, False), (False, False), (False, True)))
    pts1 = torch.rand(2000, 3, generator=g) * 6 - 3
    add("p1d", dict(vsize_xyz=[0.05], coors_range_xyz=[-2, 2], num_point_features=2, max_num_voxels=60,
                    max_num_points_per_voxel=8), pts1)
    add("p2d", dict(vsize_xyz=[0.1, 0.2], coors_range_xyz=[-2, -2, 2, 2], num_point_features=3,
                    max_num_voxels=2000, max_num_points_per_voxel=2), pts1)
    pts4 = torch.rand(2500, 6, generator=g) * 4.4 - 2.2
    add("p4d", dict(vsize_xyz=[0.5, 0.4, 0.3, 0.2], coors_range_xyz=[-2, -2, -2, -2, 2, 2, 2, 2],
                    num_point_features=5, max_num_voxels=4000, max_num_points_per_voxel=3), pts4)
    edge = torch.tensor([[0.0, 0.0, 0.0], [1.0, 1.0, 1.0], [0.1, 0.1, 0.1], [0.30000001, 0.2, 0.1],
                         [0.3, 0.3, 0.3], [-1e-9, 0.5, 0.5], [0.99999994, 0.99999994, 0.99999994],
                         [float("nan"), 0.5, 0.5], [0.5, float("inf"), 0.5], [0.7, 0.7, 0.7], [0.7, 0.7, 0.7],
                         [0.1, 0.1, 0.1]], dtype=torch.float32)
    add("edges", dict(vsize_xyz=[0.1, 0.1, 0.1], coors_range_xyz=[0, 0, 0, 1, 1, 1], num_point_features=3,
                      max_num_voxels=100, max_num_points_per_voxel=2), edge, calls=((True, False), (True, True)))
    add("all_outside", dict(vsize_xyz=[0.1, 0.1, 0.1], coors_range_xyz=[0, 0, 0, 1, 1, 1], num_point_features=3,
                            max_num_voxels=10, max_num_points_per_voxel=2), edge[:2] + 5.0)
    torch.save(dict(frozen=frozen, generated=cases), OUT)
    print("wrote", OUT, OUT.stat().st_size, "bytes;", len(frozen), "frozen +", len(cases), "generated cases")


if __name__ == "__main__":
    main()
