"""Utility namespace (reference: spconv_triton/utils/__init__.py): the
``Point2Voxel{CPU,GPU}{1-4}d`` classes.  The CPU classes exist for import
compatibility and raise when constructed: voxelisation runs on CUDA only."""

from contextlib import AbstractContextManager

import torch

CPU_ONLY_BUILD = False


class nullcontext(AbstractContextManager):
    """Context manager that does no additional processing."""

    def __init__(self, enter_result=None):
        self.enter_result = enter_result

    def __enter__(self):
        return self.enter_result

    def __exit__(self, *excinfo):
        pass


from spconv_triton_b200.pytorch.utils import PointToVoxel as _PointToVoxel  # noqa: E402


def _make_p2v(ndim: int, device_type: str):
    class _Point2Voxel(_PointToVoxel):
        def __init__(self, vsize_xyz, coors_range_xyz, num_point_features, max_num_voxels,
                     max_num_points_per_voxel):
            if len(vsize_xyz) != ndim:
                raise AssertionError
            super().__init__(vsize_xyz, coors_range_xyz, num_point_features, max_num_voxels,
                             max_num_points_per_voxel, device=torch.device(device_type))

    _Point2Voxel.__name__ = _Point2Voxel.__qualname__ = f"Point2Voxel{device_type.upper()}{ndim}d"
    return _Point2Voxel


Point2VoxelCPU1d = _make_p2v(1, "cpu")
Point2VoxelCPU2d = _make_p2v(2, "cpu")
Point2VoxelCPU3d = _make_p2v(3, "cpu")
Point2VoxelCPU4d = _make_p2v(4, "cpu")
Point2VoxelGPU1d = _make_p2v(1, "cuda")
Point2VoxelGPU2d = _make_p2v(2, "cuda")
Point2VoxelGPU3d = _make_p2v(3, "cuda")
Point2VoxelGPU4d = _make_p2v(4, "cuda")
