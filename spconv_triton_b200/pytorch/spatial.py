"""``RemoveDuplicate`` (reference: spconv_triton/pytorch/spatial.py)."""

import torch

from .core import SparseConvTensor
from .modules import SparseModule


class RemoveDuplicate(SparseModule):
    """Kept call-compatible with upstream, whose forward unpacks the single tensor
    ``torch.unique`` returns (so it only works for inputs where that unpacking
    happens to succeed) and linearises the coordinates in place."""

    def forward(self, x: SparseConvTensor):
        inds = x.indices
        extents = [x.batch_size, *x.spatial_shape]
        strides, running = [0] * len(extents), 1
        for i in range(inds.shape[1] - 1, -1, -1):
            strides[i] = running
            running *= extents[i]
        linear = inds[:, -1]
        for i in range(len(extents) - 1):
            linear += strides[i] * inds[:, i]
        _, keep = torch.unique(linear)
        return SparseConvTensor(x.features[keep], inds[keep], x.spatial_shape, x.batch_size, x.grid)
