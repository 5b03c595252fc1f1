"""Point cloud voxelisation (reference: spconv_triton/pytorch/utils.py).

``PointToVoxel`` keeps the reference's constructor, persistent buffers, return
values and first-come-first-served semantics; the work is done by
``spc_voxelize`` of the CUDA library (hash table + prefix sum + one stable
radix sort) and its results equal the reference's bit for bit.  CUDA tensors
only: there is no CPU path.
"""

from __future__ import annotations

import ctypes

import torch

from spconv_triton_b200 import _lib


class PointToVoxel:
    """WARNING: you MUST construct PointToVoxel AFTER set device."""

    def __init__(self, vsize_xyz: list[float], coors_range_xyz: list[float], num_point_features: int,
                 max_num_voxels: int, max_num_points_per_voxel: int,
                 device: torch.device = torch.device("cpu:0")):
        self.ndim = len(vsize_xyz)
        self.device = torch.device(device)
        self.num_point_features = num_point_features
        self.max_num_voxels = max_num_voxels
        self.max_num_points_per_voxel = max_num_points_per_voxel
        if self.device.type != "cuda":
            raise NotImplementedError("spconv_triton_b200 voxelises on CUDA devices only (no CPU path)")

        cmin = coors_range_xyz[: self.ndim]
        cmax = coors_range_xyz[self.ndim:]
        grid_size_xyz = [round((cmax[i] - cmin[i]) / vsize_xyz[i]) for i in range(self.ndim)]
        self._vsize_xyz = list(vsize_xyz)
        self._grid_size_xyz = grid_size_xyz
        self._coors_range_xyz = list(coors_range_xyz)
        # public metadata is stored reversed (z, y, x), as upstream (reference: utils.py:44-52)
        self.vsize = list(reversed(vsize_xyz))
        self.grid_size = list(reversed(grid_size_xyz))
        self.coors_range = list(reversed(cmin)) + list(reversed(cmax))
        stride = [1] * self.ndim
        for i in range(self.ndim - 2, -1, -1):
            stride[i] = stride[i + 1] * self.grid_size[i + 1]
        self.grid_stride = stride

        self.voxels = torch.zeros([max_num_voxels, max_num_points_per_voxel, num_point_features],
                                  dtype=torch.float32, device=self.device)
        self.indices = torch.zeros([max_num_voxels, self.ndim], dtype=torch.int32, device=self.device)
        self.num_per_voxel = torch.zeros([max_num_voxels], dtype=torch.int32, device=self.device)

    def __call__(self, pc: torch.Tensor, clear_voxels: bool = True, empty_mean: bool = False):
        res = self.generate_voxel_with_id(pc, clear_voxels, empty_mean)
        return res[0], res[1], res[2]

    def generate_voxel_with_id(self, pc: torch.Tensor, clear_voxels: bool = True, empty_mean: bool = False):
        """``(voxels [M, P, F], indices [M, ndim] zyx, num_per_voxel [M], pc_voxel_id [N])``
        (reference: utils.py:72-163)."""
        if pc.device.type != self.device.type:
            raise AssertionError("your pc device is wrong")
        if pc.dtype != torch.float32:
            raise NotImplementedError("points must be float32 (voxel boundaries are computed in the points' dtype)")
        if pc.dim() != 2 or pc.shape[1] < max(self.ndim, self.num_point_features):
            raise AssertionError("points must be [N, >= max(ndim, num_point_features)]")
        pc = pc.contiguous()
        n = int(pc.shape[0])
        lib = _lib.load()
        nd = self.ndim
        cmin = (ctypes.c_float * nd)(*[float(v) for v in self._coors_range_xyz[:nd]])
        vsize = (ctypes.c_float * nd)(*[float(v) for v in self._vsize_xyz])
        grid = (ctypes.c_int32 * nd)(*[int(v) for v in self._grid_size_xyz])
        with torch.no_grad(), torch.cuda.device(pc.device):
            pc_voxel_id = torch.empty([n], dtype=torch.int64, device=pc.device)
            nbytes = int(lib.spc_voxelize_workspace_bytes(n, self.max_num_voxels))
            if nbytes == 0:
                raise _lib.SpconvB200Error("voxelize: sizes out of range")
            ws = torch.empty(nbytes, dtype=torch.uint8, device=pc.device)
            num = ctypes.c_int64(0)
            _lib.check(lib.spc_voxelize(
                _lib.ptr(pc) if n else None, n, int(pc.stride(0)) if n else max(nd, self.num_point_features), nd,
                self.num_point_features, cmin, vsize, grid, self.max_num_voxels, self.max_num_points_per_voxel,
                int(bool(clear_voxels)), int(bool(empty_mean)), _lib.ptr(ws), nbytes, _lib.ptr(self.voxels),
                _lib.ptr(self.indices), _lib.ptr(self.num_per_voxel), _lib.ptr(pc_voxel_id) if n else None,
                ctypes.byref(num), _lib.current_stream(pc.device)))
            m = int(num.value)
            return (self.voxels[:m].clone(), self.indices[:m].clone(), self.num_per_voxel[:m].clone(), pc_voxel_id)


def gather_features_by_pc_voxel_id(seg_res_features: torch.Tensor, pc_voxel_id: torch.Tensor,
                                   invalid_value: int | float = 0):
    """Per-voxel results back onto the points they came from; points without a
    voxel receive ``invalid_value`` (reference: utils.py:166-192)."""
    if seg_res_features.device != pc_voxel_id.device:
        pc_voxel_id = pc_voxel_id.to(seg_res_features.device)
    shape = (pc_voxel_id.shape[0], *seg_res_features.shape[1:])
    res = torch.full(shape, invalid_value, dtype=seg_res_features.dtype, device=seg_res_features.device)
    valid = torch.nonzero(pc_voxel_id != -1).view(-1)
    res[valid] = seg_res_features[pc_voxel_id[valid]]
    return res
