"""Multi-branch helpers (reference: spconv_triton/pytorch/tables.py)."""

from __future__ import annotations

import torch

from .core import SparseConvTensor
from .modules import SparseModule


def _check_aligned(tensors, what):
    first = tensors[0]
    for t in tensors:
        same = (t.spatial_shape == first.spatial_shape and t.batch_size == first.batch_size
                and t.features.shape[1] == first.features.shape[1]
                and t.indices.shape[0] == first.indices.shape[0])
        if not same:
            raise AssertionError(what)


def _like_first(tensors, features):
    first = tensors[0]
    out = SparseConvTensor(features, first.indices, first.spatial_shape, first.batch_size, first.grid,
                           first.voxel_num, first.indice_dict)
    # bookkeeping objects are taken from the second input, as upstream does
    out.benchmark_record = tensors[1].benchmark_record
    out.thrust_allocator = tensors[1].thrust_allocator
    out._timer = tensors[1]._timer
    return out


class JoinTable(SparseModule):
    """Concatenate the channels of tensors that share one set of indices."""

    def forward(self, inputs: list[SparseConvTensor]):
        _check_aligned(inputs, "you can't use JoinTable in two sptensor with different indices.")
        return _like_first(inputs, torch.cat([t.features for t in inputs], 1))

    def input_spatial_size(self, out_size):
        return out_size


class AddTable(SparseModule):
    """Sum the features of tensors that share one set of indices."""

    def forward(self, inputs: list[SparseConvTensor]):
        _check_aligned(inputs, "you can't use AddTable in two sptensor with different indices. "
                               "use AddTableMisaligned instead.")
        return _like_first(inputs, sum([t.features for t in inputs]))

    def input_spatial_size(self, out_size):
        return out_size


class AddTableMisaligned(SparseModule):
    """Add sparse tensors of one shape but different voxel sets (tables.py:78-85 of the reference)."""

    def forward(self, inputs: list[SparseConvTensor]):
        from . import functional as F

        return F.sparse_add_hash_based(*inputs)

    def input_spatial_size(self, out_size):
        return out_size


class ConcatTable(SparseModule):
    """Apply every child to the same input and return the list of results."""

    def forward(self, x):
        return [module(x) for module in self._modules.values()]

    def add(self, module):
        self._modules[str(len(self._modules))] = module
        return self

    def input_spatial_size(self, out_size):
        return self._modules["0"].input_spatial_size(out_size)
