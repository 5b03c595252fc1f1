"""Implicit gather-GEMM through the C ABI.

Same three entry points and arguments as the reference module
spconv_triton/pytorch/_impl/gemm.py (conv_forward :501, conv_backward_input
:571, conv_backward_weight :634); precision policy as :456-483.
"""

from __future__ import annotations

import torch

from spconv_triton_b200 import _lib, constants

from .pairs import rowmajor_of

# Which kernels the GEMM entry points may use: SPC_GEMM_AUTO (tcgen05 whenever
# the shape allows), SPC_GEMM_SIMT or SPC_GEMM_TCGEN05.  Tests flip this.
GEMM_PATH = _lib.SPC_GEMM_AUTO


def check_device_status(device=None):
    """Synchronise the current stream and raise if a kernel recorded that one of
    its bounded device-side waits expired."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    with torch.cuda.device(dev):
        _lib.check(_lib.load().spc_check_device_status(_lib.current_stream(dev)))


def _precision(t: torch.Tensor) -> int:
    # TF32 only for fp32 inputs and only while the live flag is set (gemm.py:460-463)
    if t.dtype == torch.float32 and bool(constants.SPCONV_ALLOW_TF32):
        return _lib.SPC_PREC_TF32
    return _lib.SPC_PREC_IEEE


def _rowmajor(pair_table, t):
    """Row-major table copy for the tensor-core kernels (the CUDA-core kernels,
    which serve IEEE fp32, do not use it, so none is built for them)."""
    rm = getattr(pair_table, "_spc_rowmajor", None)
    if rm is None and (t.dtype in (torch.float16, torch.bfloat16) or _precision(t) == _lib.SPC_PREC_TF32):
        rm = rowmajor_of(pair_table)
    return rm


def _order(kv, pair_mask, mask_argsort):
    # gemm.py:486-498: the mask-sorted row order applies only to single-word masks
    if pair_mask is not None and mask_argsort is not None and 1 < kv <= 32:
        return mask_argsort if mask_argsort.is_contiguous() else mask_argsort.contiguous()
    return None


def conv_forward(features, filters_krsc, pair_fwd, n_out, bias=None, out_dtype=None, pair_mask=None,
                 mask_argsort=None, fp32_accum=None, epilogue=None):
    """out [n_out, K] = gather-GEMM of features [N, C] with filters [K, kv, C].

    ``epilogue`` (not in the reference): ``(scale, shift, act, alpha)`` applied
    while the rows are stored -- out = act((acc + bias) * scale + shift) with
    fp32 ``scale``/``shift`` of shape [K] (or both None) and ``act`` one of the
    ``_lib.SPC_ACT_*`` codes.

    ``fp32_accum`` is accepted for signature parity: 16-bit inputs always
    accumulate in fp32 here, which the reference treats as the accurate
    default (gemm.py:15-22)."""
    if not features.is_cuda:
        raise AssertionError
    k_out, kv, c_in = filters_krsc.shape
    if out_dtype is None:
        out_dtype = features.dtype
    dev = features.device
    with torch.cuda.device(dev):
        out = torch.empty((n_out, k_out), dtype=out_dtype, device=dev)
        if n_out == 0:
            return out
        feats = features.contiguous()
        w = filters_krsc.contiguous()
        if w.dtype != feats.dtype:
            w = w.to(feats.dtype)
        b = None
        if bias is not None:
            b = bias.contiguous()
            if b.dtype != feats.dtype:
                b = b.to(feats.dtype)
        pf = pair_fwd if pair_fwd.is_contiguous() else pair_fwd.contiguous()
        order = _order(kv, pair_mask, mask_argsort)
        scale = shift = None
        act, alpha = _lib.SPC_ACT_NONE, 0.0
        if epilogue is not None:
            scale, shift, act, alpha = epilogue
        _lib.check(_lib.load().spc_conv_forward(
            _lib.ptr(feats), _lib.ptr(w), _lib.ptr(b), _lib.ptr(pf), _lib.ptr(_rowmajor(pair_fwd, feats)), _lib.ptr(order),
            _lib.ptr(out),
            feats.shape[0], n_out, c_in, k_out, kv, _lib.dtype_code(feats.dtype), _lib.dtype_code(out_dtype),
            _precision(feats), GEMM_PATH, _lib.ptr(scale), _lib.ptr(shift), int(act), float(alpha),
            _lib.current_stream(dev)))
    return out


def conv_backward_input(grad_out, filters_krsc, pair_bwd, n_in, pair_mask=None, mask_argsort=None,
                        fp32_accum=None):
    """din [n_in, C] = sum_k grad_out[pair_bwd[k, :]] @ W[k]."""
    k_out, kv, c_in = filters_krsc.shape
    dev = grad_out.device
    with torch.cuda.device(dev):
        din = torch.empty((n_in, c_in), dtype=grad_out.dtype, device=dev)
        if n_in == 0:
            return din
        g = grad_out.contiguous()
        w = filters_krsc.contiguous()
        if w.dtype != g.dtype:
            w = w.to(g.dtype)
        pb = pair_bwd if pair_bwd.is_contiguous() else pair_bwd.contiguous()
        order = _order(kv, pair_mask, mask_argsort)
        _lib.check(_lib.load().spc_conv_backward_input(
            _lib.ptr(g), _lib.ptr(w), _lib.ptr(pb), _lib.ptr(_rowmajor(pair_bwd, g)), _lib.ptr(order), _lib.ptr(din), n_in, g.shape[0], c_in,
            k_out, kv, _lib.dtype_code(g.dtype), _precision(g), GEMM_PATH, _lib.current_stream(dev)))
    return din


def conv_backward_weight(features, grad_out, pair_fwd, weight_shape_krsc, fp32_accum=None):
    """dW [K, kv, C] (contiguous, grad_out.dtype)."""
    k_out, kv, c_in = (int(v) for v in weight_shape_krsc)
    n_out = int(grad_out.shape[0])
    dev = grad_out.device
    with torch.cuda.device(dev):
        dw = torch.empty((k_out, kv, c_in), dtype=grad_out.dtype, device=dev)
        if n_out == 0 or kv == 0:
            dw.zero_()
            return dw
        feats = features.contiguous()
        g = grad_out.contiguous()
        if feats.dtype != g.dtype:
            feats = feats.to(g.dtype)
        pf = pair_fwd if pair_fwd.is_contiguous() else pair_fwd.contiguous()
        lib = _lib.load()
        nbytes = int(lib.spc_conv_backward_weight_workspace_bytes(n_out, c_in, k_out, kv))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        _lib.check(lib.spc_conv_backward_weight(
            _lib.ptr(feats), _lib.ptr(g), _lib.ptr(pf), _lib.ptr(dw), _lib.ptr(ws), ws.numel(),
            feats.shape[0], n_out, c_in, k_out, kv, _lib.dtype_code(g.dtype), _precision(g), GEMM_PATH,
            _lib.current_stream(dev)))
    return dw
