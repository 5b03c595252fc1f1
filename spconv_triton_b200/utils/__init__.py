"""``spconv_triton_b200.utils``: the eight ``Point2Voxel{CPU,GPU}{1..4}d`` names
of the reference's utils namespace (spconv_triton/utils/__init__.py) over the
CUDA voxeliser of this package.  The CPU names exist so that imports keep
working; constructing one raises, because voxelisation here runs on CUDA only."""

from contextlib import nullcontext  # noqa: F401  (re-exported, as the reference's namespace does)

import torch

from spconv_triton_b200.pytorch.utils import PointToVoxel as _PointToVoxel

CPU_ONLY_BUILD = False


class _FixedRank(_PointToVoxel):
    """PointToVoxel bound to one dimensionality and one device type (class attributes)."""

    _ndim = 0
    _device_type = "cuda"

    def __init__(self, vsize_xyz, coors_range_xyz, num_point_features, max_num_voxels, max_num_points_per_voxel):
        if len(vsize_xyz) != self._ndim:
            raise AssertionError
        super().__init__(vsize_xyz, coors_range_xyz, num_point_features, max_num_voxels, max_num_points_per_voxel,
                         device=torch.device(self._device_type))


for _dev in ("cpu", "cuda"):
    for _nd in (1, 2, 3, 4):
        _name = f"Point2Voxel{'CPU' if _dev == 'cpu' else 'GPU'}{_nd}d"
        globals()[_name] = type(_name, (_FixedRank,), {"_ndim": _nd, "_device_type": _dev, "__module__": __name__})
del _dev, _nd, _name
