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


def _rowmajor(pair_table, t, tensor_cores=None):
    """Row-major table copy for the tensor-core kernels (the CUDA-core kernels
    do not use it, so none is built for them)."""
    rm = getattr(pair_table, "_spc_rowmajor", None)
    if tensor_cores is None:
        tensor_cores = t.dtype in (torch.float16, torch.bfloat16) or _precision(t) == _lib.SPC_PREC_TF32
    if rm is None and tensor_cores:
        rm = rowmajor_of(pair_table)
    return rm


# fp32 layers on the tensor cores.  With SPCONV_ALLOW_TF32 the operands are rounded to TF32
# (round to nearest, as the reference's tl.dot does) and multiplied once; without it (IEEE mode,
# the reference's default) each operand is split into two TF32 numbers and the reduction runs over
# [hi | lo | hi] . [hi | hi | lo], which carries fp32 accuracy at three times the TF32 work.  Set to
# False to keep IEEE-mode fp32 layers on the CUDA cores.
FP32_ON_TENSOR_CORES = True
# The tensor cores add into their fp32 accumulator with truncation, so the error of the split path
# grows with the number of accumulated terms: measured 4e-6 of the largest output at kv * c_in = 864,
# 9e-6 at 1728, 1.7e-5 at 3456 (about 5e-9 per term).  IEEE mode promises 1e-5, so longer
# reductions stay on the CUDA cores (IEEE fused multiply-add, 1e-6).
FP32_SPLIT_MAX_REDUCTION = 1024


def _fp32_plan(n_dim, r_dim, kv):
    """(mode for the gathered operand, mode for the weight, reduction multiplier) if an fp32 layer
    with ``n_dim`` outputs and reduction ``r_dim`` per kernel offset can run on the tcgen05
    kernels, else None."""
    if GEMM_PATH == _lib.SPC_GEMM_SIMT or n_dim % 16 or not 16 <= n_dim <= 256 or r_dim % 8:
        return None
    if bool(constants.SPCONV_ALLOW_TF32):
        return _lib.SPC_TF32_ROUND, _lib.SPC_TF32_ROUND, 1
    if FP32_ON_TENSOR_CORES and kv * r_dim <= FP32_SPLIT_MAX_REDUCTION:
        return _lib.SPC_TF32_SPLIT_A, _lib.SPC_TF32_SPLIT_B, 3
    return None


def _prepared_rows(x, mode, mult):
    out = torch.empty((x.shape[0], mult * x.shape[1]), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().spc_tf32_prepare(_lib.ptr(x), _lib.ptr(out), x.shape[0], x.shape[1], mode,
                                            _lib.current_stream(x.device)))
    return out


def _prepared_weight(w, transpose, mode, mult):
    """Prepared copy of the KRSC weight, remembered on the tensor until it changes."""
    owner = w._base if w._base is not None else w  # the layer's parameter when ``w`` is a reshaped view of it
    key = (w._version, w.data_ptr(), tuple(w.shape), bool(transpose), mode)
    cache = getattr(owner, "_spc_tf32", None)
    if cache is None:
        cache = {}
        try:
            owner._spc_tf32 = cache
        except AttributeError:
            pass
    hit = cache.get((bool(transpose), mode))
    if hit is not None and hit[0] == key:
        return hit[1]
    k_out, kv, c_in = w.shape
    shape = (c_in, kv, mult * k_out) if transpose else (k_out, kv, mult * c_in)
    out = torch.empty(shape, dtype=torch.float32, device=w.device)
    _lib.check(_lib.load().spc_tf32_prepare_weight(_lib.ptr(w), _lib.ptr(out), k_out, kv, c_in, int(bool(transpose)),
                                                   mode, _lib.current_stream(w.device)))
    cache[(bool(transpose), mode)] = (key, out)
    return out


def _order(kv, pair_mask, mask_argsort):
    # gemm.py:486-498: the mask-sorted row order applies only to single-word masks
    if pair_mask is not None and mask_argsort is not None and 1 < kv <= 32:
        return mask_argsort if mask_argsort.is_contiguous() else mask_argsort.contiguous()
    return None


def conv_forward(features, filters_krsc, pair_fwd, n_out, bias=None, out_dtype=None, pair_mask=None,
                 mask_argsort=None, fp32_accum=None, epilogue=None, residual=None):
    """out [n_out, K] = gather-GEMM of features [N, C] with filters [K, kv, C].

    ``epilogue`` (not in the reference): ``(scale, shift, act, alpha)`` applied
    while the rows are stored -- out = act((acc + bias) * scale + shift) with
    fp32 ``scale``/``shift`` of shape [K] (or both None) and ``act`` one of the
    ``_lib.SPC_ACT_*`` codes.

    ``residual`` (not in the reference): a tensor [n_out, K] of the output dtype
    added to the result while the rows are stored (a residual connection in the
    same pass; the reference adds ``add_input`` afterwards, conv.py:503-511).

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
        precision, tensor_cores = _precision(feats), None
        plan = _fp32_plan(k_out, c_in, kv) if feats.dtype == torch.float32 and out_dtype == torch.float32 else None
        if plan is not None:
            feats = _prepared_rows(feats, plan[0], plan[2])
            w = _prepared_weight(w, False, plan[1], plan[2])
            c_in, precision, tensor_cores = plan[2] * c_in, _lib.SPC_PREC_TF32, True
        if residual is not None:
            if residual.shape != out.shape or residual.dtype != out_dtype or residual.device != dev:
                raise ValueError("residual must have the shape, dtype and device of the output")
            residual = residual.contiguous()
        _lib.check(_lib.load().spc_conv_forward_residual(
            _lib.ptr(feats), _lib.ptr(w), _lib.ptr(b), _lib.ptr(pf), _lib.ptr(_rowmajor(pair_fwd, feats, tensor_cores)),
            _lib.ptr(order), _lib.ptr(out),
            feats.shape[0], n_out, c_in, k_out, kv, _lib.dtype_code(feats.dtype), _lib.dtype_code(out_dtype),
            precision, GEMM_PATH, _lib.ptr(scale), _lib.ptr(shift), int(act), float(alpha), _lib.ptr(residual),
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
        plan = _fp32_plan(c_in, k_out, kv) if g.dtype == torch.float32 else None
        if plan is not None:
            # the input gradient as a forward convolution of grad_out with the transposed weight
            gp = _prepared_rows(g, plan[0], plan[2])
            wt = _prepared_weight(w, True, plan[1], plan[2])
            _lib.check(_lib.load().spc_conv_forward(
                _lib.ptr(gp), _lib.ptr(wt), None, _lib.ptr(pb), _lib.ptr(_rowmajor(pair_bwd, g, True)), _lib.ptr(order),
                _lib.ptr(din), g.shape[0], n_in, plan[2] * k_out, c_in, kv, _lib.SPC_F32, _lib.SPC_F32,
                _lib.SPC_PREC_TF32, GEMM_PATH, None, None, _lib.SPC_ACT_NONE, 0.0, _lib.current_stream(dev)))
            return din
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
