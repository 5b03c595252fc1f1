"""spconv_triton_b200: B200 (sm_100a) implementation of the sparse-convolution
hot path behind the ``spconv_triton.pytorch`` API.

    import spconv_triton_b200.pytorch as spconv

Rulebook generation, the implicit gather-GEMM (forward, input and weight
gradients) and sparse max/avg pooling run as hand-written CUDA kernels in
``csrc/libspconv_b200.so`` (C ABI in ``include/spconv_b200.h``).  There is no
Triton, no CPU fallback and no alternative backend.
"""

from . import constants
from .core import AlgoHint, ConvAlgo

__version__ = "1.0.0+b200"

# Version triple of the upstream API this package is call-compatible with.
SPCONV_VERSION_NUMBERS = [2, 3, 8]

__all__ = ["AlgoHint", "ConvAlgo", "constants", "SPCONV_VERSION_NUMBERS", "__version__"]
