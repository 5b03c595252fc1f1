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
                act_beta: float = 0.0, act_type=_NO_ACT, residual: torch.Tensor | None = None):
        # ``residual`` (not in the reference): added to the output inside the kernel's store; its
        # gradient is the output gradient
        out, mask_out, mask_width = ops.implicit_gemm(
            features, filters, pair_fwd, pair_mask_fwd_splits, mask_argsort_fwd_splits, num_activate_out,
            masks, is_train, is_subm, timer, fp32_accum, bias, act_alpha, act_beta, act_type,
            _residual=residual)
        ctx.has_residual = residual is not None
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
            is_subm=e["is_subm"], timer=e["timer"], fp32_accum=e["fp32_accum"],
            _need_din=ctx.needs_input_grad[0])
        return (din, dw) + (None,) * 16 + ((grad_output if ctx.has_residual else None),)


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


# ---- misaligned sparse add --------------------------------------------------------------------
_MAX_INT32 = 2147483647


def _indice_to_scalar(indices: torch.Tensor, shape: list[int]):
    """Row-major linear index of [N, len(shape)] coordinates (functional.py:415-426 of the reference)."""
    if indices.shape[1] != len(shape):
        raise AssertionError
    stride = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        stride[i] = stride[i + 1] * shape[i + 1]
    scalar_inds = indices[:, -1].clone()
    for i in range(len(shape) - 1):
        scalar_inds += stride[i] * indices[:, i]
    return scalar_inds.contiguous()


class _RowsScatterAdd(Function):
    """out[rows_k[i], :] += features_k[i, :] over all operands k, and the coordinates with them.

    args = (rows_0.., indices_0.., features_0..), ``n_tens`` of each.  The gradient of operand k
    is the gather grad_out[rows_k]."""

    @staticmethod
    def forward(ctx, count, n_tens, *args):
        from spconv_triton_b200 import _lib

        rows, idxs, feats = args[:n_tens], args[n_tens:2 * n_tens], args[2 * n_tens:]
        first = feats[0]
        channels, width = int(first.shape[1]), int(idxs[0].shape[1])
        out = torch.zeros([count, channels], dtype=first.dtype, device=first.device)
        out_idx = torch.zeros([count, width], dtype=idxs[0].dtype, device=first.device)
        lib = _lib.load()
        code = _lib.dtype_code(first.dtype)
        with torch.cuda.device(first.device):
            stream = _lib.current_stream(first.device)
            for r, ix, f in zip(rows, idxs, feats, strict=True):
                f, ix = f.contiguous(), ix.contiguous()
                _lib.check(lib.spc_rows_scatter_add(_lib.ptr(f), _lib.ptr(r), int(f.shape[0]), channels, code, count,
                                                    _lib.ptr(out), _lib.ptr(ix), width, _lib.ptr(out_idx), stream))
        ctx.save_for_backward(*rows)
        ctx.meta = (n_tens, channels, code)
        ctx.mark_non_differentiable(out_idx)
        return out, out_idx

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_out, _grad_idx):
        from spconv_triton_b200 import _lib

        n_tens, channels, code = ctx.meta
        grad_out = grad_out.contiguous()
        lib = _lib.load()
        grads = []
        with torch.cuda.device(grad_out.device):
            stream = _lib.current_stream(grad_out.device)
            for k, r in enumerate(ctx.saved_tensors):
                if not ctx.needs_input_grad[2 + 2 * n_tens + k]:
                    grads.append(None)
                    continue
                g = torch.empty([r.shape[0], channels], dtype=grad_out.dtype, device=grad_out.device)
                _lib.check(lib.spc_rows_gather(_lib.ptr(grad_out), _lib.ptr(r), int(r.shape[0]), channels, code,
                                               int(grad_out.shape[0]), _lib.ptr(g), stream))
                grads.append(g)
        return (None, None, *([None] * (2 * n_tens)), *grads)


def _sparse_add_cuda(tens):
    import ctypes

    from spconv_triton_b200 import _lib

    from .core import SparseConvTensor
    from .hash import HashTable

    table_size = 0
    max_num_indices = 0
    max_num_indices_idx = 0
    for i, ten in enumerate(tens):
        if ten.spatial_shape != tens[0].spatial_shape:
            raise AssertionError
        if ten.batch_size != tens[0].batch_size:
            raise AssertionError
        if ten.features.shape[1] != tens[0].features.shape[1]:
            raise AssertionError
        table_size += ten.features.shape[0]
        if max_num_indices < ten.features.shape[0]:
            max_num_indices_idx = i
            max_num_indices = ten.features.shape[0]
    first = tens[0]
    if not first.features.is_cuda:
        raise NotImplementedError("spconv_triton_b200 sparse add is CUDA only")
    shape = [first.batch_size, *first.spatial_shape]
    whole_shape = int(np.prod(shape))
    k_type = torch.int64 if whole_shape >= _MAX_INT32 else torch.int32
    # sized for every row of every operand (the reference doubles this; capacity only), so no insert can fill it
    table = HashTable(first.features.device, k_type, torch.int32, max(table_size, 1))
    table._key_bits = max(1, (whole_shape - 1).bit_length())
    lib = _lib.load()
    shape_arr = (ctypes.c_int64 * len(shape))(*[int(v) for v in shape])
    scalars = []
    with torch.cuda.device(first.features.device):
        stream = _lib.current_stream(first.features.device)
        for ten in tens:
            indices = ten.indices.contiguous()
            if indices.shape[1] != len(shape):
                raise AssertionError
            scalar = torch.empty(indices.shape[0], dtype=k_type, device=indices.device)
            _lib.check(lib.spc_coords_to_keys(_lib.ptr(indices), int(indices.shape[0]), len(shape), shape_arr,
                                              scalar.element_size(), _lib.ptr(scalar), stream))
            scalars.append(scalar)
            table._insert_unchecked(scalar)
    count_val = table._items(0, None, None, 0)  # assign_arange_ without the device round trip of its count
    rows = [table.query(scalar)[0] for scalar in scalars]
    out_features, out_indices = _RowsScatterAdd.apply(
        count_val, len(tens), *rows, *[t.indices for t in tens], *[t.features for t in tens])
    res = SparseConvTensor(out_features, out_indices, first.spatial_shape, first.batch_size, benchmark=first.benchmark)
    if count_val == max_num_indices:
        res.indice_dict = tens[max_num_indices_idx].indice_dict
    res.benchmark_record = first.benchmark_record
    res._timer = first._timer
    res.thrust_allocator = first.thrust_allocator
    return res


def sparse_add_hash_based(*tens):
    """Sum of sparse tensors whose voxel sets differ (functional.py:429-490 of the reference).

    The union of the coordinates is numbered through a GPU hash table in ascending order of the
    linear coordinate (what the reference's sorted table gives), then every operand's rows are
    accumulated into their numbered rows by one kernel per operand."""
    return _sparse_add_cuda(tens)


def sparse_add(*tens):
    """Same sum; the reference goes through torch.sparse coalescing (functional.py:493-535), whose
    result rows are in the same ascending coordinate order, so both names share one CUDA path."""
    return _sparse_add_cuda(tens)
