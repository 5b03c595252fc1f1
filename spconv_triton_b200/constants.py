"""Configuration constants, same names and defaults as the reference's
spconv_triton/constants.py.

Read by this package:
  SPCONV_SAVED_WEIGHT_LAYOUT (env)  checkpoint weight layout handled by the
                                    conv load hook
  SPCONV_FX_TRACE_MODE (env)        skip SparseConvTensor argument checks
  SPCONV_DO_SORT (env)              default of ``do_sort`` in pair generation
  SPCONV_ALLOW_TF32                 live switch: fp32 GEMMs use TF32 tensor cores
  SPCONV_FOLD_BN_RELU (env)         fold inference BatchNorm + ReLU into the conv kernel
  SPCONV_RULEBOOK_RUNAHEAD (env)    build the next layer's rulebook beside the current GEMM
  SPCONV_NATIVE_SEQUENCE (env)      run an inference SparseSequential of convolutions as one library call
  SPCONV_ALLOW_FP16_ACCUM (env)     accepted; 16-bit GEMMs always accumulate in
                                    fp32 on B200 (full rate, more accurate)
Everything else is kept only so that ``from ...constants import X`` works.
"""

import os
from pathlib import Path

PACKAGE_ROOT = Path(__file__).parent.resolve()

SAVED_WEIGHT_LAYOUT = os.getenv("SPCONV_SAVED_WEIGHT_LAYOUT", "")
if SAVED_WEIGHT_LAYOUT not in ("", "KRSC", "RSKC", "RSCK"):
    raise AssertionError("please set SAVED_WEIGHT_LAYOUT to KRSC, RSKC or RSCK")

SPCONV_FX_TRACE_MODE = os.getenv("SPCONV_FX_TRACE_MODE", "0") == "1"
SPCONV_DO_SORT = os.getenv("SPCONV_DO_SORT", "1") == "1"
SPCONV_USE_DIRECT_TABLE = True
SPCONV_DEBUG_WEIGHT = False
SPCONV_ALLOW_TF32 = False
SPCONV_ALLOW_FP16_ACCUM = os.getenv("SPCONV_ALLOW_FP16_ACCUM", "0") == "1"
# Not in the reference.  In evaluation mode SparseSequential runs
# [sparse conv, BatchNorm1d, ReLU] as one kernel (normalisation folded into the
# GEMM's store).  Read at call time; set to False for the unfused modules.
SPCONV_FOLD_BN_RELU = os.getenv("SPCONV_FOLD_BN_RELU", "1") == "1"
# Not in the reference.  SparseSequential builds the rulebook of the next layer on
# a second CUDA stream while the GEMM of the current layer runs (same results).
# Read at call time.
SPCONV_RULEBOOK_RUNAHEAD = os.getenv("SPCONV_RULEBOOK_RUNAHEAD", "1") == "1"
# Not in the reference.  An inference pass of a SparseSequential made only of implicit-gemm
# convolutions (+ BatchNorm1d + ReLU) runs as one call into the library (pytorch/sequence.py)
# instead of layer by layer from Python; same kernels and results.  Read at call time.
SPCONV_NATIVE_SEQUENCE = os.getenv("SPCONV_NATIVE_SEQUENCE", "1") == "1"
NDIM_DONT_CARE = 3

ALL_WEIGHT_IS_KRSC = True
FILTER_HWIO = False
DISABLE_JIT = False
EDITABLE_INSTALLED = False
BOOST_ROOT = None
SPCONV_DEBUG_SAVE_PATH = ""
SPCONV_BWD_SPLITK = [1, 2, 4, 8, 16, 32, 64]
SPCONV_DIRECT_TABLE_HASH_SIZE_SCALE = 1.1
SPCONV_INT8_DEBUG = False
PACKAGE_NAME = "spconv_triton_b200"
SPCONV_DEBUG_CPP_ONLY = False
SPCONV_DEBUG_NVRTC_KERNELS = False
SPCONV_CPP_INDICE_PAIRS = False
SPCONV_CPP_INDICE_PAIRS_IGEMM = False
SPCONV_CPP_GEMM = False


class AllocKeys:
    """Allocator dictionary keys of the upstream API (unused: outputs are torch tensors)."""


for _k in ("PairBwd IndiceNumPerLoc PairMask MaskArgSort OutIndices PairFwd PairMaskBwd MaskArgSortBwd "
           "MaskOutputFwd OutFeatures Features Filters OutBp DIn DFilters InpBuffer OutBuffer "
           "IndicePairsUniq IndicePairsUniqBackup HashKOrKV HashV ThrustTemp TightUniqueCount").split():
    setattr(AllocKeys, _k, _k)
del _k
