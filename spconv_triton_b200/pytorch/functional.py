"""Autograd functions over the primitive operators (the layer the reference
implements in spconv_triton/pytorch/functional.py).

Forward passes are AMP-aware: inside ``torch.autocast`` their floating-point
inputs are cast to fp16 (``custom_fwd(cast_inputs=torch.float16)``), and every
backward is once-differentiable.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.amp as amp
from torch.autograd import Function
from torch.autograd.function import once_differentiable

from spconv_triton_b200.compat import tv
from spconv_triton_b200.tools import CUDAKernelTimer

from . import ops

_fwd = amp.custom_fwd(cast_inputs=torch.float16, device_type="cuda")
_bwd = amp.custom_bwd(device_type="cuda")
_NO_ACT = tv.gemm.Activation.None_
_NO_TIMER = CUDAKernelTimer(False)


def _native_conv_function(name: str, inverse: bool, subm: bool):
    """Builds the autograd Function of one Native-format convolution flavour;
    the three flavours differ only in the (inverse, subm) flags handed to the
    operator (reference: functional.py:51-114, 117-182, 264-329)."""

    class _Fn(Function):
        @staticmethod
        @_fwd
        def forward(ctx, features, filters, indice_pairs, indice_pair_num, num_activate_out, algo,
                    timer: CUDAKernelTimer = _NO_TIMER, bias: torch.Tensor | None = None,
                    act_alpha: float = 0.0, act_beta: float = 0.0, act_type=_NO_ACT):
            ctx.save_for_backward(indice_pairs, indice_pair_num, features, filters)
            ctx.algo, ctx.timer = algo, timer
            return ops.indice_conv(features, filters, indice_pairs, indice_pair_num, num_activate_out,
                                   inverse, subm, algo=algo, timer=timer, bias=bias, act_alpha=act_alpha,
                                   act_beta=act_beta, act_type=act_type)

        @staticmethod
        @once_differentiable
        @_bwd
        def backward(ctx, grad_output):
            indice_pairs, indice_pair_num, features, filters = ctx.saved_tensors
            din, dw = ops.indice_conv_backward(features, filters, grad_output, indice_pairs, indice_pair_num,
                                               inverse, subm, algo=ctx.algo, timer=ctx.timer)
            return (din, dw) + (None,) * 9

    _Fn.__name__ = _Fn.__qualname__ = name
    return _Fn


SparseConvFunction = _native_conv_function("SparseConvFunction", inverse=False, subm=False)
SparseInverseConvFunction = _native_conv_function("SparseInverseConvFunction", inverse=True, subm=False)
SubMConvFunction = _native_conv_function("SubMConvFunction", inverse=False, subm=True)


class SparseImplicitGemmFunction(Function):
    """Implicit-gemm convolution (reference: functional.py:185-261)."""

    @staticmethod
    @_fwd
    def forward(ctx, features, filters, pair_fwd, pair_bwd, pair_mask_fwd_splits, pair_mask_bwd_splits,
                mask_argsort_fwd_splits, mask_argsort_bwd_splits, num_activate_out: int,
                masks: list[np.ndarray], is_train: bool, is_subm: bool, timer: CUDAKernelTimer = _NO_TIMER,
                fp32_accum: bool | None = None, bias: torch.Tensor | None = None, act_alpha: float = 0.0,
                act_beta: float = 0.0, act_type=_NO_ACT):
        out, mask_out, mask_width = ops.implicit_gemm(
            features, filters, pair_fwd, pair_mask_fwd_splits, mask_argsort_fwd_splits, num_activate_out,
            masks, is_train, is_subm, timer, fp32_accum, bias, act_alpha, act_beta, act_type)
        ctx.save_for_backward(features, filters, pair_fwd, pair_bwd)
        ctx.extra = dict(pair_mask_fwd_splits=pair_mask_fwd_splits, pair_mask_bwd_splits=pair_mask_bwd_splits,
                         mask_argsort_fwd_splits=mask_argsort_fwd_splits,
                         mask_argsort_bwd_splits=mask_argsort_bwd_splits, mask_output_fwd=mask_out,
                         masks=masks, mask_width=mask_width, is_subm=is_subm, timer=timer,
                         fp32_accum=fp32_accum)
        return out

    @staticmethod
    @once_differentiable
    @_bwd
    def backward(ctx, grad_output):
        features, filters, pair_fwd, pair_bwd = ctx.saved_tensors
        e = ctx.extra
        din, dw = ops.implicit_gemm_backward(
            features, filters, grad_output, pair_fwd, pair_bwd, e["pair_mask_fwd_splits"],
            e["pair_mask_bwd_splits"], e["mask_argsort_fwd_splits"], e["mask_argsort_bwd_splits"],
            mask_output_fwd=e["mask_output_fwd"], masks=e["masks"], mask_width=e["mask_width"],
            is_subm=e["is_subm"], timer=e["timer"], fp32_accum=e["fp32_accum"])
        return (din, dw) + (None,) * 16


class SparseMaxPoolFunction(Function):
    """Native-format max pool (reference: functional.py:332-350)."""

    @staticmethod
    @_fwd
    def forward(ctx, features, indice_pairs, indice_pair_num, num_activate_out):
        out = ops.indice_maxpool(features, indice_pairs, indice_pair_num, num_activate_out)
        ctx.save_for_backward(indice_pairs, indice_pair_num, features, out)
        return out

    @staticmethod
    @once_differentiable
    @_bwd
    def backward(ctx, grad_output):
        indice_pairs, indice_pair_num, features, out = ctx.saved_tensors
        return ops.indice_maxpool_backward(features, out, grad_output, indice_pairs, indice_pair_num), None, None, None


class SparseMaxPoolImplicitGemmFunction(Function):
    """Implicit-gemm max pool (reference: functional.py:353-377)."""

    @staticmethod
    @_fwd
    def forward(ctx, features, indice_pairs_fwd, indice_pairs_bwd, num_activate_out: int):
        out = ops.indice_maxpool_implicit_gemm(features, indice_pairs_fwd, num_activate_out)
        ctx.save_for_backward(indice_pairs_bwd, features, out)
        return out

    @staticmethod
    @once_differentiable
    @_bwd
    def backward(ctx, grad_output):
        indice_pairs_bwd, features, out = ctx.saved_tensors
        return ops.indice_maxpool_implicit_gemm_backward(features, out, grad_output, indice_pairs_bwd), None, None, None


class SparseAvgPoolImplicitGemmFunction(Function):
    """Implicit-gemm average pool; the per-row input count is saved for the
    backward (reference: functional.py:380-405)."""

    @staticmethod
    @_fwd
    def forward(ctx, features, indice_pairs_fwd, indice_pairs_bwd, num_activate_out: int, calc_count):
        out, count = ops.indice_avgpool_implicit_gemm(features, indice_pairs_fwd, num_activate_out, calc_count)
        ctx.save_for_backward(indice_pairs_bwd, features, out, count)
        return out

    @staticmethod
    @once_differentiable
    @_bwd
    def backward(ctx, grad_output):
        indice_pairs_bwd, _features, _out, count = ctx.saved_tensors
        return ops.indice_avgpool_implicit_gemm_backward(grad_output, indice_pairs_bwd, count), None, None, None, None


indice_conv = SparseConvFunction.apply
implicit_gemm = SparseImplicitGemmFunction.apply
indice_inverse_conv = SparseInverseConvFunction.apply
indice_subm_conv = SubMConvFunction.apply
indice_maxpool = SparseMaxPoolFunction.apply
indice_maxpool_implicit_gemm = SparseMaxPoolImplicitGemmFunction.apply
indice_avgpool_implicit_gemm = SparseAvgPoolImplicitGemmFunction.apply
