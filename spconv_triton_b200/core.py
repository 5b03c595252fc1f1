"""Algorithm enums (same members and values as the reference's spconv_triton/core.py)."""

from enum import Enum

from .constants import NDIM_DONT_CARE  # noqa: F401  (re-export)


class ConvAlgo(Enum):
    Native = 0
    MaskImplicitGemm = 1
    MaskSplitImplicitGemm = 2


class AlgoHint(Enum):
    NoHint = 0
    Fowrard = 1  # spelling is part of the upstream API
    BackwardInput = 2
    BackwardWeight = 4
