"""Primitive operators with the call signatures of ``spconv.pytorch.ops``.

This is the layer the reference implements in spconv_triton/pytorch/ops.py;
each function adapts its arguments and calls one of the three ``_impl``
modules, which here are ctypes wrappers over libspconv_b200.so.
"""

from __future__ import annotations

import numpy as np
import torch

from spconv_triton_b200.compat import tv
from spconv_triton_b200.constants import (  # noqa: F401  (re-exports of the upstream module)
    ALL_WEIGHT_IS_KRSC,
    FILTER_HWIO,
    SPCONV_DO_SORT,
    SPCONV_USE_DIRECT_TABLE,
    AllocKeys,
)
from spconv_triton_b200.core import AlgoHint, ConvAlgo  # noqa: F401
from spconv_triton_b200.tools import CPU_ONLY_BUILD, CUDAKernelTimer, nullcontext  # noqa: F401

from ._impl import gemm as _gemm
from ._impl import pairs as _pairs
from ._impl import pool as _pool
from ._impl.pairs import get_conv_output_size, get_deconv_output_size
from .core import ThrustSortAllocator
from .cppcore import get_current_stream  # noqa: F401

INT32_MAX = 2147483647
DEBUG = False
DEBUG_INT64_HASH_K = False

__all__ = [
    "ConvAlgo", "get_conv_output_size", "get_deconv_output_size", "get_indice_pairs",
    "get_indice_pairs_implicit_gemm", "global_pool_rearrange", "implicit_gemm", "implicit_gemm_backward",
    "indice_avgpool_implicit_gemm", "indice_avgpool_implicit_gemm_backward", "indice_conv",
    "indice_conv_backward", "indice_maxpool", "indice_maxpool_backward", "indice_maxpool_implicit_gemm",
    "indice_maxpool_implicit_gemm_backward", "maximum_value_int_",
]

_NO_ACT = tv.gemm.Activation.None_


def _require_cuda(t: torch.Tensor, msg: str = ""):
    if not t.is_cuda:
        raise AssertionError(msg)


def _reject_int8(t: torch.Tensor):
    if t.dtype in (torch.int8, torch.qint8):
        raise NotImplementedError("int8 is not supported by spconv_triton")


_INPLACE_ACTIVATIONS = {
    "None_": lambda t, alpha: t,
    "ReLU": lambda t, alpha: t.relu_(),
    "Sigmoid": lambda t, alpha: t.sigmoid_(),
    "LeakyReLU": lambda t, alpha: torch.nn.functional.leaky_relu_(t, alpha),
}


def _apply_act_inplace(out: torch.Tensor, act_type, act_alpha: float, act_beta: float):
    """The activation enum applied to ``out`` in place (the reference applies it
    after its kernel the same way, spconv_triton/pytorch/ops.py:63-73; here it is
    only used where the activation is not fused into the GEMM's store)."""
    name = getattr(act_type, "name", "None_")
    fn = _INPLACE_ACTIVATIONS.get(name)
    if fn is None:
        raise NotImplementedError(f"activation {name} not supported")
    return fn(out, act_alpha)


def _act_code(act_type) -> int:
    name = getattr(act_type, "name", "None_")
    try:
        return {"None_": 0, "ReLU": 1, "Sigmoid": 2, "LeakyReLU": 3}[name]
    except KeyError:
        raise NotImplementedError(f"activation {name} not supported") from None


def _filters_krsc(filters: torch.Tensor):
    """[K, *ksize, C] -> contiguous [K, kv, C]."""
    return filters.reshape(filters.shape[0], -1, filters.shape[-1]).contiguous()


# ---- rulebooks -----------------------------------------------------------------------------

def get_indice_pairs(indices, batch_size, spatial_shape, algo, ksize, stride, padding, dilation, out_padding,
                     subm: bool = False, transpose: bool = False, num_out_act_bound: int = -1):
    """Native rulebook -> ``(out_inds, pair [2,kv,N], indice_num_per_loc)``; the
    bound is not honoured by this format (reference: ops.py:86-113)."""
    if algo != ConvAlgo.Native:
        raise AssertionError("TODO")
    return _pairs.native_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation,
                               out_padding, subm, transpose)


def get_indice_pairs_implicit_gemm(indices, batch_size, spatial_shape, algo, ksize, stride, padding, dilation,
                                   out_padding, subm: bool = False, transpose: bool = False,
                                   is_train: bool = True, alloc: ThrustSortAllocator | None = None,
                                   timer: CUDAKernelTimer = CUDAKernelTimer(False),
                                   num_out_act_bound: int = -1, direct_table: bool = SPCONV_USE_DIRECT_TABLE,
                                   do_sort: bool = SPCONV_DO_SORT):
    """Implicit-gemm rulebook, 9-tuple (reference: ops.py:116-155)."""
    _require_cuda(indices, "implicit gemm only support gpu tensors")
    if algo not in (ConvAlgo.MaskImplicitGemm, ConvAlgo.MaskSplitImplicitGemm):
        raise AssertionError("TODO")
    return _pairs.igemm_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation,
                              out_padding, subm, transpose, is_train,
                              algo == ConvAlgo.MaskSplitImplicitGemm, do_sort, num_out_act_bound)


# ---- convolution ---------------------------------------------------------------------------

def indice_conv(features, filters, indice_pairs, indice_pair_num, num_activate_out, inverse: bool = False,
                subm: bool = False, algo: ConvAlgo = ConvAlgo.Native,
                timer: CUDAKernelTimer = CUDAKernelTimer(False), bias: torch.Tensor | None = None,
                act_alpha: float = 0.0, act_beta: float = 0.0, act_type=_NO_ACT):
    """Native-format forward (reference: ops.py:163-194)."""
    features = features.contiguous()
    _reject_int8(features)
    pf, _ = _pairs.native_pair_to_tables(indice_pairs, indice_pair_num, features.shape[0], num_activate_out,
                                         inverse, need_bwd=False)
    out = _gemm.conv_forward(features, _filters_krsc(filters), pf, num_activate_out, bias=bias)
    return _apply_act_inplace(out, act_type, act_alpha, act_beta)


def fused_indice_conv(features, filters, bias, indice_pairs, indice_pair_num, num_activate_out, inverse, subm):
    raise NotImplementedError


def indice_conv_backward(features, filters, out_bp, indice_pairs, indice_pair_num, inverse: bool = False,
                         subm: bool = False, algo: ConvAlgo = ConvAlgo.Native,
                         timer: CUDAKernelTimer = CUDAKernelTimer(False)):
    """Native-format backward -> ``(din, dfilters)`` (reference: ops.py:210-234)."""
    features = features.contiguous()
    out_bp = out_bp.contiguous()
    w = _filters_krsc(filters)
    pf, pb = _pairs.native_pair_to_tables(indice_pairs, indice_pair_num, features.shape[0], out_bp.shape[0],
                                          inverse)
    din = _gemm.conv_backward_input(out_bp, w, pb, features.shape[0])
    dw = _gemm.conv_backward_weight(features, out_bp, pf, w.shape)
    return din, dw.reshape(filters.shape)


def _single_split_mask(pair_mask_splits, mask_argsort_splits, masks):
    """1-D (mask, argsort) of the single-split case, else (None, None)
    (reference: ops.py:237-256)."""
    if len(masks) != 1 or len(pair_mask_splits) != 1 or len(mask_argsort_splits) != 1:
        return None, None
    pm, ar = pair_mask_splits[0], mask_argsort_splits[0]
    if pm.numel() == 0 or ar.numel() == 0:
        return None, None
    return (pm[:, 0] if pm.dim() == 2 else pm), ar


def implicit_gemm(features, filters, pair_fwd, pair_mask_fwd_splits, mask_argsort_fwd_splits,
                  num_activate_out: int, masks: list[np.ndarray], is_train: bool, is_subm: bool,
                  timer: CUDAKernelTimer = CUDAKernelTimer(False), fp32_accum: bool | None = None,
                  bias: torch.Tensor | None = None, act_alpha: float = 0.0, act_beta: float = 0.0,
                  act_type=_NO_ACT, output_scale: float = 1.0, scale: torch.Tensor | None = None,
                  output_add: torch.Tensor | None = None, output_add_scale: float = 0.0,
                  output_dtype: torch.dtype | None = None, _bn_fold=None, _residual=None):
    """Implicit-gemm forward -> ``(out, mask_output_fwd, mask_width)``
    (reference: ops.py:259-305).  The activation is applied inside the kernel's
    store; ``_bn_fold = (scale, shift)`` (fp32 [K], not in the reference) folds
    an inference BatchNorm in front of it; ``_residual`` (not in the reference)
    is added to the result in the same store."""
    if output_add is not None and features.dtype != torch.qint8:
        raise AssertionError("fused residual add only support int8")
    _reject_int8(features)
    features = features.contiguous()
    pm, ar = _single_split_mask(pair_mask_fwd_splits, mask_argsort_fwd_splits, masks)
    scale, shift = _bn_fold if _bn_fold is not None else (None, None)
    out = _gemm.conv_forward(features, _filters_krsc(filters), pair_fwd, num_activate_out, bias=bias,
                             out_dtype=output_dtype, pair_mask=pm, mask_argsort=ar, fp32_accum=fp32_accum,
                             epilogue=(scale, shift, _act_code(act_type), float(act_alpha)), residual=_residual)
    return out, torch.Tensor(), -1


def implicit_gemm_backward(features, filters, grad_output, pair_fwd, pair_bwd, pair_mask_fwd_splits,
                           pair_mask_bwd_splits, mask_argsort_fwd_splits, mask_argsort_bwd_splits,
                           mask_output_fwd, masks: list[np.ndarray], mask_width: int, is_subm: bool,
                           timer: CUDAKernelTimer = CUDAKernelTimer(False), fp32_accum: bool | None = None,
                           _need_din: bool = True):
    """Implicit-gemm backward -> ``(din, dfilters)`` (reference: ops.py:308-347).
    ``_need_din=False`` (not in the reference) skips the input gradient, which autograd does not
    ask for at the first layer of a network; ``din`` is then None."""
    features = features.contiguous()
    grad_output = grad_output.contiguous()
    w = _filters_krsc(filters)
    pm, ar = _single_split_mask(pair_mask_bwd_splits, mask_argsort_bwd_splits, masks)
    din = None
    if _need_din:
        din = _gemm.conv_backward_input(grad_output, w, pair_bwd, features.shape[0], pair_mask=pm,
                                        mask_argsort=ar, fp32_accum=fp32_accum)
    dw = _gemm.conv_backward_weight(features, grad_output, pair_fwd, w.shape, fp32_accum=fp32_accum)
    return din, dw.reshape(filters.shape)


# ---- pooling -------------------------------------------------------------------------------

def indice_maxpool(features, indice_pairs, indice_pair_num, num_activate_out):
    features = features.contiguous()
    pf, _ = _pairs.native_pair_to_tables(indice_pairs, indice_pair_num, features.shape[0],
                                         int(num_activate_out), False, need_bwd=False)
    return _pool.maxpool_forward(features, pf, int(num_activate_out))


def indice_maxpool_backward(features, out_features, out_bp, indice_pairs, indice_pair_num):
    _, pb = _pairs.native_pair_to_tables(indice_pairs, indice_pair_num, features.shape[0],
                                         out_features.shape[0], False)
    return _pool.maxpool_backward(features, out_features, out_bp, pb)


def indice_maxpool_implicit_gemm(features, indice_pairs, num_activate_out):
    _require_cuda(features)
    return _pool.maxpool_forward(features.contiguous(), indice_pairs, int(num_activate_out))


def indice_maxpool_implicit_gemm_backward(features, out_features, out_bp, indice_pairs):
    _require_cuda(features)
    return _pool.maxpool_backward(features, out_features, out_bp, indice_pairs)


def indice_avgpool_implicit_gemm(features, indice_pairs, num_activate_out, calc_count: bool):
    _require_cuda(features)
    out, count = _pool.avgpool_forward(features.contiguous(), indice_pairs, int(num_activate_out), calc_count)
    return out, (count if calc_count else torch.Tensor())


def indice_avgpool_implicit_gemm_backward(out_bp, indice_pairs, count_out):
    _require_cuda(out_bp)
    return _pool.avgpool_backward(out_bp, indice_pairs, count_out)


# ---- misc ----------------------------------------------------------------------------------

def maximum_value_int_(ten: torch.Tensor, value: int):
    ten.clamp_(min=int(value))


def global_pool_rearrange(coords: torch.Tensor, batch_size: int):
    """Per-sample row lists: ``out_indices[b, :counts[b]]`` are the rows of sample b."""
    n = coords.shape[0]
    device = coords.device
    out_indices = torch.empty((batch_size, n), dtype=torch.int32, device=device)
    if n == 0:
        return out_indices, torch.zeros((batch_size,), dtype=torch.int32, device=device)
    b = coords[:, 0].long()
    counts = torch.bincount(b, minlength=batch_size)
    order = torch.argsort(b, stable=True)
    starts = torch.cumsum(counts, 0) - counts
    sorted_b = b[order]
    out_indices[sorted_b, torch.arange(n, device=device) - starts[sorted_b]] = order.to(torch.int32)
    return out_indices, counts.to(torch.int32)
