"""Stand-in for the small part of ``cumm.tensorview`` that leaks into layer
constructors: ``tv.gemm.Activation`` (reference: spconv_triton/compat.py)."""

from enum import Enum
from types import SimpleNamespace


class Activation(Enum):
    None_ = 0
    ReLU = 1
    Sigmoid = 2
    LeakyReLU = 3


tv = SimpleNamespace(gemm=SimpleNamespace(Activation=Activation))
