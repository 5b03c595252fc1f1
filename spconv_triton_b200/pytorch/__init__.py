"""Public PyTorch API: ``import spconv_triton_b200.pytorch as spconv``."""

from . import functional, hash, ops
from .conv import (
    SparseConv1d, SparseConv2d, SparseConv3d, SparseConv4d,
    SparseConvTranspose1d, SparseConvTranspose2d, SparseConvTranspose3d, SparseConvTranspose4d,
    SparseInverseConv1d, SparseInverseConv2d, SparseInverseConv3d, SparseInverseConv4d,
    SubMConv1d, SubMConv2d, SubMConv3d, SubMConv4d,
)
from .core import SparseConvTensor
from .identity import Identity
from .modules import (
    SparseBatchNorm, SparseIdentity, SparseModule, SparseReLU, SparseSequential,
    assign_name_for_sparse_modules,
)
from .ops import ConvAlgo
from .pool import (
    SparseAvgPool1d, SparseAvgPool2d, SparseAvgPool3d, SparseGlobalAvgPool, SparseGlobalMaxPool,
    SparseMaxPool1d, SparseMaxPool2d, SparseMaxPool3d, SparseMaxPool4d,
)
from .tables import AddTable, AddTableMisaligned, ConcatTable, JoinTable


class ToDense(SparseModule):
    """SparseConvTensor -> dense channels-first tensor."""

    def forward(self, x: SparseConvTensor):
        return x.dense()


class RemoveGrid(SparseModule):
    """Drops the pre-allocated grid buffer."""

    def forward(self, x: SparseConvTensor):
        x.grid = None
        return x
