"""ctypes binding of libspconv_b200.so (the C ABI declared in include/spconv_b200.h).

There is no fallback: if the library has not been built, importing a symbol
from here raises, and every operator of the package fails with it.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libspconv_b200.so"

SPC_MAX_NDIM = 4
SPC_F16, SPC_BF16, SPC_F32, SPC_F64 = 0, 1, 2, 3
SPC_PREC_IEEE, SPC_PREC_TF32 = 0, 1
SPC_TF32_ROUND, SPC_TF32_SPLIT_A, SPC_TF32_SPLIT_B = 0, 1, 2
SPC_ACT_NONE, SPC_ACT_RELU, SPC_ACT_SIGMOID, SPC_ACT_LEAKY_RELU = 0, 1, 2, 3
SPC_GEMM_AUTO, SPC_GEMM_SIMT, SPC_GEMM_TCGEN05, SPC_GEMM_TCGEN05_CPASYNC = 0, 1, 2, 3
(SPC_OK, SPC_ERR_INVALID_ARGUMENT, SPC_ERR_CUDA, SPC_ERR_WORKSPACE_TOO_SMALL, SPC_ERR_HASH_TABLE_FULL,
 SPC_ERR_UNSUPPORTED, SPC_ERR_DEVICE_WAIT_EXPIRED, SPC_ERR_SIZE_LIMIT) = range(8)

_I4 = c_int32 * SPC_MAX_NDIM


class Geometry(ctypes.Structure):
    """Mirror of ``spc_geometry``."""

    _fields_ = [
        ("ndim", c_int32),
        ("batch_size", c_int32),
        ("in_shape", _I4),
        ("out_shape", _I4),
        ("ksize", _I4),
        ("stride", _I4),
        ("padding", _I4),
        ("dilation", _I4),
        ("subm", c_int32),
        ("transpose", c_int32),
    ]


def _pad4(vals, fill):
    vals = [int(v) for v in vals]
    return _I4(*(vals + [fill] * (SPC_MAX_NDIM - len(vals))))


def make_geometry(batch_size, in_shape, out_shape, ksize, stride, padding, dilation, subm, transpose):
    g = Geometry()
    g.ndim = len(in_shape)
    g.batch_size = int(batch_size)
    g.in_shape = _pad4(in_shape, 1)
    g.out_shape = _pad4(out_shape, 1)
    g.ksize = _pad4(ksize, 1)
    g.stride = _pad4(stride, 1)
    g.padding = _pad4(padding, 0)
    g.dilation = _pad4(dilation, 1)
    g.subm = int(bool(subm))
    g.transpose = int(bool(transpose))
    return g


_P = c_void_p
_PROTOTYPES = {
    "spc_version": (c_int, []),
    "spc_last_error": (c_char_p, []),
    "spc_launch_count": (ctypes.c_longlong, []),
    "spc_check_device_status": (c_int, [_P]),
    "spc_post_device_status": (c_int, [_P, _P]),
    "spc_tf32_prepare": (c_int, [_P, _P, c_int64, c_int, c_int, _P]),
    "spc_sequence_forward": (c_int, [_P, c_int, _P, _P, c_int64, c_int, _P, c_size_t, _P, _P, _P, _P, _P]),
    "spc_tf32_prepare_weight": (c_int, [_P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "spc_conv_output_size": (c_int, [c_int, POINTER(c_int32), POINTER(c_int32), POINTER(c_int32),
                                     POINTER(c_int32), POINTER(c_int32), POINTER(c_int32)]),
    "spc_deconv_output_size": (c_int, [c_int, POINTER(c_int32), POINTER(c_int32), POINTER(c_int32),
                                       POINTER(c_int32), POINTER(c_int32), POINTER(c_int32), POINTER(c_int32)]),
    "spc_rulebook_workspace_bytes": (c_size_t, [POINTER(Geometry), c_int64]),
    "spc_rulebook_prepare": (c_int, [POINTER(Geometry), _P, c_int64, _P, c_size_t, POINTER(c_int64), _P]),
    "spc_rulebook_igemm": (c_int, [POINTER(Geometry), _P, c_int64, c_int64, _P, c_size_t, _P, _P, _P, _P, _P,
                                   _P, _P, POINTER(c_uint32), c_int, c_int, _P, _P, _P]),
    "spc_rulebook_igemm_backward": (c_int, [POINTER(Geometry), _P, c_int64, c_int64, _P, c_size_t, _P, _P, _P,
                                            POINTER(c_uint32), c_int, c_int, _P, _P]),
    "spc_pairs_to_rowmajor": (c_int, [_P, c_int, c_int64, _P, _P]),
    "spc_dense_scatter": (c_int, [_P, _P, c_int64, c_int, c_int, c_int, POINTER(ctypes.c_int32), c_int, c_int, _P, _P]),
    "spc_dense_gather": (c_int, [_P, _P, c_int64, c_int, c_int, c_int, POINTER(ctypes.c_int32), c_int, c_int, _P, _P]),
    "spc_from_dense_workspace_bytes": (c_size_t, [c_int64]),
    "spc_from_dense_count": (c_int, [_P, c_int64, c_int, c_int, c_int, _P, c_size_t, POINTER(c_int64), _P]),
    "spc_from_dense_indices": (c_int, [_P, c_int64, c_int, POINTER(ctypes.c_int32), _P, _P]),
    "spc_global_pool_workspace_bytes": (c_size_t, [c_int, c_int]),
    "spc_global_pool": (c_int, [_P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P]),
    "spc_hash_bytes": (c_size_t, [c_int64]),
    "spc_hash_clear": (c_int, [_P, c_int64, _P]),
    "spc_hash_insert": (c_int, [_P, c_int64, _P, c_int, _P, c_int, c_int64, ctypes.c_uint64, _P]),
    "spc_hash_counters": (c_int, [_P, c_int64, POINTER(c_int64), POINTER(c_int64), _P]),
    "spc_hash_query": (c_int, [_P, c_int64, _P, c_int, c_int64, _P, c_int, _P, _P]),
    "spc_hash_update": (c_int, [_P, c_int64, _P, c_int, _P, c_int, c_int64, _P, _P]),
    "spc_hash_items_workspace_bytes": (c_size_t, [c_int64]),
    "spc_hash_items": (c_int, [_P, c_int64, c_int64, c_int, c_int, _P, c_size_t, _P, c_int, _P, c_int, c_int64, _P]),
    "spc_coords_to_keys": (c_int, [_P, c_int64, c_int, POINTER(c_int64), c_int, _P, _P]),
    "spc_rows_scatter_add": (c_int, [_P, _P, c_int64, c_int, c_int, c_int64, _P, _P, c_int, _P, _P]),
    "spc_rows_gather": (c_int, [_P, _P, c_int64, c_int, c_int, c_int64, _P, _P]),
    "spc_voxelize_workspace_bytes": (c_size_t, [c_int64, c_int64]),
    "spc_voxelize": (c_int, [_P, c_int64, c_int, c_int, c_int, POINTER(ctypes.c_float), POINTER(ctypes.c_float),
                             POINTER(ctypes.c_int32), c_int64, c_int, c_int, c_int, _P, c_size_t, _P, _P, _P, _P,
                             POINTER(c_int64), _P]),
    "spc_rulebook_native": (c_int, [POINTER(Geometry), _P, c_int64, c_int64, _P, c_size_t, _P, _P, _P, _P]),
    "spc_native_to_tables": (c_int, [_P, c_int, c_int64, c_int, _P, c_int64, _P, c_int64, _P]),
    "spc_conv_forward": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, _P, _P, c_int, ctypes.c_float, _P]),
    "spc_conv_forward_needs_colmajor": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "spc_conv_forward_residual": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                          c_int, c_int, c_int, _P, _P, c_int, ctypes.c_float, _P, _P]),
    "spc_conv_backward_input": (c_int, [_P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int,
                                        c_int, c_int, _P]),
    "spc_conv_backward_weight_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int]),
    "spc_conv_backward_weight": (c_int, [_P, _P, _P, _P, _P, c_size_t, c_int64, c_int64, c_int, c_int, c_int,
                                         c_int, c_int, c_int, _P]),
    "spc_conv_backward_weight_noalloc_max_bytes": (c_size_t, []),
    "spc_conv_backward_weight_noalloc": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, _P]),
    "spc_maxpool_forward": (c_int, [_P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "spc_maxpool_backward": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "spc_avgpool_forward": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "spc_avgpool_backward": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
}

# Entry points that exist in the header but may be added after the first build.
_OPTIONAL = {}

_lib = None


def exported_symbols():
    """Names every build of the library must export."""
    return sorted(_PROTOTYPES)


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built. "
            "Run `python -m spconv_triton_b200.csrc.build` (needs nvcc); there is no CPU fallback."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in {**_PROTOTYPES, **_OPTIONAL}.items():
        if name in _OPTIONAL and not hasattr(lib, name):
            continue
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


class SpconvB200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"libspconv_b200 status {status}: {message}")
        self.status = status


def check(status):
    if status != 0:
        msg = load().spc_last_error()
        raise SpconvB200Error(status, msg.decode() if msg else "")


# ---- device status mailbox -------------------------------------------------------------------
# Kernels of the library record failures they cannot raise themselves (a bounded wait that
# expired, an index row outside the grid met by a submanifold rulebook, which has no host read)
# in a per-device status word.  A forward pass ends by queueing a copy of that word into a
# page-locked host word (no wait); the next forward pass on that device starts by looking at
# the host word and raises if it is set.
_mailboxes: dict = {}


def status_mailbox(index: int):
    """(torch tensor [1] int32, numpy view) shared with the device through spc_post_device_status."""
    import torch

    box = _mailboxes.get(index)
    if box is None:
        t = torch.zeros(1, dtype=torch.int32)
        if torch.cuda.is_available():
            t = t.pin_memory()
        box = (t, t.numpy())
        _mailboxes[index] = box
    return box


def post_device_status(device) -> None:
    """Queue the copy of ``device``'s status word into its mailbox on the current stream."""
    import torch

    index = device.index if device.index is not None else torch.cuda.current_device()
    t, _ = status_mailbox(index)
    with torch.cuda.device(index):
        check(load().spc_post_device_status(c_void_p(t.data_ptr()), current_stream(device)))


def raise_posted_status(device=None) -> None:
    """Raise SpconvB200Error if a status posted by an earlier pass has arrived (never waits)."""
    import torch

    if device is None or device.index is None:
        index = torch.cuda.current_device() if torch.cuda.is_available() else 0
    else:
        index = device.index
    box = _mailboxes.get(index)
    if box is None or box[1][0] == 0:
        return
    code = int(box[1][0])
    box[1][0] = 0
    if torch.cuda.is_available():
        with torch.cuda.device(index):
            load().spc_check_device_status(current_stream(torch.device("cuda", index)))  # clears the word
    text = ("an index row outside batch_size / spatial_shape was met by a rulebook kernel (the row got no pairs)"
            if code == SPC_ERR_INVALID_ARGUMENT else
            "a bounded device-side wait expired in a kernel of an earlier pass: its output is incomplete")
    raise SpconvB200Error(code, text + "; reported by an earlier forward pass on this device")


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


_DTYPES = None


def dtype_code(dtype):
    global _DTYPES
    if _DTYPES is None:
        import torch

        _DTYPES = {torch.float16: SPC_F16, torch.bfloat16: SPC_BF16, torch.float32: SPC_F32,
                   torch.float64: SPC_F64}
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise NotImplementedError(f"dtype {dtype} is not supported by spconv_triton_b200") from None


def current_stream(device):
    import torch

    return c_void_p(torch.cuda.current_stream(device).cuda_stream)
