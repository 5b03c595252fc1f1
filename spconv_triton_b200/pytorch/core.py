"""SparseConvTensor and the rulebook cache entries kept in its ``indice_dict``.

Attribute names and behaviour follow the reference's
spconv_triton/pytorch/core.py so that user models run unchanged.
"""

from __future__ import annotations

from typing import Any, Union

import numpy as np
import torch

from spconv_triton_b200.constants import SPCONV_FX_TRACE_MODE
from spconv_triton_b200.core import ConvAlgo
from spconv_triton_b200.tools import CUDAKernelTimer

try:
    from torch.fx import ProxyableClassMeta as SpConvTensorMeta
except Exception:  # pragma: no cover - very old torch

    class SpConvTensorMeta(type):  # type: ignore[no-redef]
        pass


class ThrustSortAllocator:
    """Constructor-compatible placeholder: scratch memory comes from torch."""

    def __init__(self, device: torch.device) -> None:
        self.alloced_objs: dict = {}
        self.device = device


class _Record:
    """Plain attribute bag; subclasses list their fields in ``_fields``."""

    _fields: tuple = ()

    def _assign(self, values: dict):
        for name in self._fields:
            setattr(self, name, values[name])


class IndiceData(_Record):
    """Native-format rulebook cached under an ``indice_key`` (reference: core.py:47-76)."""

    _fields = ("out_indices", "indices", "indice_pairs", "indice_pair_num", "spatial_shape",
               "out_spatial_shape", "is_subm", "algo", "ksize", "stride", "dilation", "padding", "voxel_num")

    def __init__(self, out_indices, indices, indice_pairs, indice_pair_num, spatial_shape, out_spatial_shape,
                 is_subm: bool, algo: ConvAlgo, ksize, stride, dilation, padding, voxel_num: Any = None):
        self._assign(locals())


class ImplicitGemmIndiceData(_Record):
    """Implicit-gemm rulebook cached under an ``indice_key`` (reference: core.py:79-120)."""

    _fields = ("out_indices", "indices", "pair_fwd", "pair_bwd", "pair_mask_fwd_splits",
               "pair_mask_bwd_splits", "mask_argsort_fwd_splits", "mask_argsort_bwd_splits", "masks",
               "spatial_shape", "out_spatial_shape", "is_subm", "algo", "ksize", "stride", "dilation",
               "padding", "in_voxel_num", "out_voxel_num")

    def __init__(self, out_indices, indices, pair_fwd, pair_bwd, pair_mask_fwd_splits, pair_mask_bwd_splits,
                 mask_argsort_fwd_splits, mask_argsort_bwd_splits, masks, spatial_shape, out_spatial_shape,
                 is_subm: bool, algo: ConvAlgo, ksize, stride, dilation, padding, in_voxel_num: Any = None,
                 out_voxel_num: Any = None):
        self._late = None
        self._assign(locals())

    # The input-side tables of a strided layer may be pending (an inference forward does
    # not build them); reading any of the three attributes builds them.
    def _resolved(self, name):
        late = self.__dict__.get("_late")
        if late is not None:
            self.__dict__["_late"] = None
            pair_bwd, pm_bwd, ma_bwd = late.get()
            self.__dict__.update(_pair_bwd=pair_bwd, _pair_mask_bwd_splits=pm_bwd, _mask_argsort_bwd_splits=ma_bwd)
        return self.__dict__[name]

    # The column-major table may be pending too (the native pass writes only the row-major copy when
    # that is all its kernels read): it is then the transpose of the copy, made when first read.
    def _resolved_fwd(self):
        d = self.__dict__
        thunk = d.get("_pair_fwd_thunk")
        if thunk is not None:
            d["_pair_fwd_thunk"] = None
            d["_pair_fwd"] = thunk()
        return d["_pair_fwd"]

    def _set_fwd(self, v):
        self.__dict__["_pair_fwd_thunk"] = None
        self.__dict__["_pair_fwd"] = v

    pair_fwd = property(_resolved_fwd, _set_fwd)

    # ... and so may the sorted masks and their argsort: the native pass orders the rows for its own
    # kernels by a different key and leaves a thunk that makes the exactly sorted pair.
    def _resolved_masks(self, name):
        d = self.__dict__
        thunk = d.get("_masks_fwd_thunk")
        if thunk is not None:
            d["_masks_fwd_thunk"] = None
            pm, ma = thunk()
            if d.get("_pair_mask_fwd_splits") is None:  # not assigned by the user in the meantime
                d["_pair_mask_fwd_splits"] = pm
            if d.get("_mask_argsort_fwd_splits") is None:
                d["_mask_argsort_fwd_splits"] = ma
        return d[name]

    pair_mask_fwd_splits = property(lambda self: self._resolved_masks("_pair_mask_fwd_splits"),
                                    lambda self, v: self.__dict__.__setitem__("_pair_mask_fwd_splits", v))
    mask_argsort_fwd_splits = property(lambda self: self._resolved_masks("_mask_argsort_fwd_splits"),
                                       lambda self, v: self.__dict__.__setitem__("_mask_argsort_fwd_splits", v))
    pair_bwd = property(lambda self: self._resolved("_pair_bwd"),
                        lambda self, v: self.__dict__.__setitem__("_pair_bwd", v))
    pair_mask_bwd_splits = property(lambda self: self._resolved("_pair_mask_bwd_splits"),
                                    lambda self, v: self.__dict__.__setitem__("_pair_mask_bwd_splits", v))
    mask_argsort_bwd_splits = property(lambda self: self._resolved("_mask_argsort_bwd_splits"),
                                       lambda self, v: self.__dict__.__setitem__("_mask_argsort_bwd_splits", v))


def register_implicit_gemm_indice_data(indice_dict, indice_key, res, indices, *, is_subm, spatial_shape,
                                       out_spatial_shape, algo, ksize, stride, dilation, padding):
    """Store the 9-tuple returned by ``ops.get_indice_pairs_implicit_gemm`` under
    ``indice_key``; a key that already exists is an error (reference: core.py:123-164)."""
    if indice_key in indice_dict:
        raise AssertionError(f"your indice key {indice_key} already exists in this sparse tensor.")
    data = ImplicitGemmIndiceData(
        res[0], indices, res[2], res[3], res[4], res[5], res[6], res[7], res[8], spatial_shape,
        out_spatial_shape, is_subm, algo, ksize, stride, dilation, padding)
    data._late = getattr(res[2], "_spc_late", None)
    indice_dict[indice_key] = data


def scatter_nd(indices, updates, shape):
    """Dense tensor of ``shape`` with ``updates`` written at ``indices`` (last
    write wins; reference: core.py:167-178)."""
    ret = torch.zeros(*shape, dtype=updates.dtype, device=updates.device)
    ndim = indices.shape[-1]
    flat = indices.view(-1, ndim)
    ret[tuple(flat[:, i] for i in range(ndim)) + (Ellipsis,)] = updates.view(
        *(list(indices.shape[:-1]) + list(shape[ndim:])))
    return ret


class SparseConvTensor(metaclass=SpConvTensorMeta):
    """features [N, C] + int32 indices [N, ndim+1] (batch index first) +
    spatial shape + batch size, plus the ``indice_dict`` rulebook cache."""

    def __init__(self, features: torch.Tensor, indices: torch.Tensor, spatial_shape, batch_size: int,
                 grid: torch.Tensor | None = None, voxel_num: torch.Tensor | None = None,
                 indice_dict: dict | None = None, benchmark: bool = False,
                 permanent_thrust_allocator: bool = False, enable_timer: bool = False,
                 force_algo: ConvAlgo | None = None):
        if not SPCONV_FX_TRACE_MODE:
            if features.ndim != 2 or indices.ndim != 2:
                raise AssertionError
            if len(spatial_shape) != indices.shape[1] - 1:
                raise AssertionError("spatial shape must equal to ndim")
            if indices.dtype != torch.int32:
                raise AssertionError("only support int32")
            if batch_size <= 0:
                raise AssertionError
        self._features = features
        self.indices = indices
        self.spatial_shape = [int(v) for v in spatial_shape]
        self.batch_size = batch_size
        self.indice_dict = {} if indice_dict is None else indice_dict
        self.grid: torch.Tensor | None = torch.Tensor() if grid is None else grid
        self.voxel_num = voxel_num
        self.benchmark = benchmark
        self.benchmark_record: dict = {}
        self.thrust_allocator = ThrustSortAllocator(features.device) if permanent_thrust_allocator else None
        self._timer = CUDAKernelTimer(enable_timer)
        self.force_algo = force_algo
        self.int8_scale: np.ndarray | None = None
        self._planner = None  # rulebook run-ahead state of the enclosing SparseSequential

    def __repr__(self):
        return f"SparseConvTensor[shape={self._features.shape}]"

    # -- features are read-only; replace_feature makes a sibling tensor -------------------------
    @property
    def features(self):
        return self._features

    @features.setter
    def features(self, val):
        raise ValueError("you can't set feature directly, use 'x = x.replace_feature(your_new_feature)'"
                         " to generate new SparseConvTensor instead.")

    def _carry_over(self, other: "SparseConvTensor") -> "SparseConvTensor":
        other.benchmark_record = self.benchmark_record
        other.thrust_allocator = self.thrust_allocator
        other._timer = self._timer
        other.force_algo = self.force_algo
        other.int8_scale = self.int8_scale
        other._planner = self._planner
        return other

    def replace_feature(self, feature: torch.Tensor):
        new = SparseConvTensor(feature, self.indices, self.spatial_shape, self.batch_size, self.grid,
                               self.voxel_num, self.indice_dict)
        new.benchmark = self.benchmark
        return self._carry_over(new)

    def shadow_copy(self) -> "SparseConvTensor":
        """New object sharing every member with this one."""
        new = SparseConvTensor(self.features, self.indices, self.spatial_shape, self.batch_size, self.grid,
                               self.voxel_num, self.indice_dict, self.benchmark)
        return self._carry_over(new)

    def select_by_index(self, valid_indices: torch.Tensor):
        # assigning to the read-only property raises, as upstream does
        new = self.shadow_copy()
        new.indices = self.indices[valid_indices]
        new.features = self.features[valid_indices]
        new.indice_dict.clear()
        return new

    def minus(self):
        return self.replace_feature(-self.features)

    @property
    def is_quantized(self):
        return self.features.dtype == torch.qint8

    def q_scale(self):
        if self.is_quantized:
            return self.features.q_scale()
        raise ValueError("sparse tensor must be quantized")

    def dequantize(self):
        return self.replace_feature(self.features.dequantize())

    @property
    def spatial_size(self):
        return np.prod(self.spatial_shape)

    def find_indice_pair(self, key) -> IndiceData | ImplicitGemmIndiceData | None:
        return None if key is None else self.indice_dict.get(key)

    @classmethod
    def from_dense(cls, x: torch.Tensor):
        """From a channel-last dense tensor [B, *spatial, C]."""
        if (x.is_cuda and 3 <= x.ndim <= 6 and x.element_size() in (1, 2, 4, 8) and not x.is_complex()
                and x.dtype != torch.bool and 0 < x.numel() and x.numel() // x.shape[-1] < 2 ** 31):
            feats, indices = _FromDense.apply(x)
            return cls(feats, indices, list(x.shape[1:-1]), x.shape[0])
        sp = x.to_sparse(x.ndim - 1)
        return cls(sp.values(), sp.indices().permute(1, 0).contiguous().int(), list(sp.shape[1:-1]),
                   sp.shape[0])

    def dense(self, channels_first: bool = True):
        """Dense ``[B, C, *spatial]`` (or ``[B, *spatial, C]``) tensor (reference:
        core.py:320-334).  CUDA features go through one zero fill and one scatter
        kernel of the library instead of scatter_nd + permute + contiguous."""
        feats = self.features
        if (feats.is_cuda and self.indices.is_cuda and feats.element_size() in (2, 4, 8) and not feats.is_complex()
                and len(self.spatial_shape) <= 4 and self.indices.shape[0] > 0):
            return _DenseScatter.apply(feats, self.indices, self.batch_size, tuple(self.spatial_shape),
                                       bool(channels_first))
        shape = [self.batch_size, *self.spatial_shape, self.features.shape[1]]
        res = scatter_nd(self.indices.to(self.features.device).long(), self.features, shape)
        if not channels_first:
            return res
        ndim = len(self.spatial_shape)
        return res.permute(0, ndim + 1, *range(1, ndim + 1)).contiguous()

    @staticmethod
    def _features_of(other):
        if not isinstance(other, (SparseConvTensor, torch.Tensor)):
            raise AssertionError
        return other if isinstance(other, torch.Tensor) else other.features

    def __add__(self, other: Union["SparseConvTensor", torch.Tensor]):
        return self.replace_feature(self.features + self._features_of(other))

    __radd__ = __add__

    def __iadd__(self, other: Union["SparseConvTensor", torch.Tensor]):
        self.features += self._features_of(other)
        return self


def _dense_call(fn_name, src, indices, batch_size, spatial_shape, channels_first, dst):
    import ctypes

    from spconv_triton_b200 import _lib

    shape = (ctypes.c_int32 * len(spatial_shape))(*[int(v) for v in spatial_shape])
    with torch.cuda.device(src.device):
        _lib.check(getattr(_lib.load(), fn_name)(
            _lib.ptr(src), _lib.ptr(indices), int(indices.shape[0]), int(src.shape[1] if fn_name == "spc_dense_scatter"
                                                                        else dst.shape[1]),
            len(spatial_shape), int(batch_size), shape, int(channels_first), src.element_size(), _lib.ptr(dst),
            _lib.current_stream(src.device)))
    return dst


class _DenseScatter(torch.autograd.Function):
    """features [N, C] -> dense; the gradient gathers the dense gradient back per row."""

    @staticmethod
    def forward(ctx, features, indices, batch_size, spatial_shape, channels_first):
        indices = indices.contiguous()
        c = features.shape[1]
        shape = [batch_size, c, *spatial_shape] if channels_first else [batch_size, *spatial_shape, c]
        out = torch.empty(shape, dtype=features.dtype, device=features.device)
        _dense_call("spc_dense_scatter", features.contiguous(), indices, batch_size, spatial_shape, channels_first, out)
        ctx.save_for_backward(indices)
        ctx.meta = (batch_size, spatial_shape, channels_first, c)
        return out

    @staticmethod
    def backward(ctx, grad):
        (indices,) = ctx.saved_tensors
        batch_size, spatial_shape, channels_first, c = ctx.meta
        gfeat = torch.empty((indices.shape[0], c), dtype=grad.dtype, device=grad.device)
        _dense_call("spc_dense_gather", grad.contiguous(), indices, batch_size, spatial_shape, channels_first, gfeat)
        return gfeat, None, None, None, None


class _FromDense(torch.autograd.Function):
    """[B, *spatial, C] -> (features [n, C], indices [n, ndim + 1]) of the cells with a non-zero
    channel, in ascending cell order (reference: core.py:296-304 through torch's to_sparse)."""

    @staticmethod
    def forward(ctx, x):
        import ctypes

        from spconv_triton_b200 import _lib

        x = x.contiguous()
        lib = _lib.load()
        spatial, c = [int(v) for v in x.shape[1:-1]], int(x.shape[-1])
        cells = x.numel() // c
        shape = (ctypes.c_int32 * len(spatial))(*spatial)
        ws = torch.empty(lib.spc_from_dense_workspace_bytes(cells), dtype=torch.uint8, device=x.device)
        count = ctypes.c_int64(0)
        with torch.cuda.device(x.device):
            stream = _lib.current_stream(x.device)
            _lib.check(lib.spc_from_dense_count(_lib.ptr(x), cells, c, x.element_size(), int(x.is_floating_point()),
                                                _lib.ptr(ws), ws.numel(), ctypes.byref(count), stream))
            n = int(count.value)
            indices = torch.empty([n, len(spatial) + 1], dtype=torch.int32, device=x.device)
            feats = torch.empty([n, c], dtype=x.dtype, device=x.device)
            if n > 0:
                _lib.check(lib.spc_from_dense_indices(_lib.ptr(ws), cells, len(spatial), shape, _lib.ptr(indices), stream))
        if n > 0:
            if x.element_size() == 1:
                feats = x.reshape(cells, c)[_cell_numbers(indices, spatial)]
            else:
                _dense_call("spc_dense_gather", x, indices, x.shape[0], spatial, False, feats)
        ctx.save_for_backward(indices)
        ctx.meta = (tuple(x.shape), spatial)
        ctx.mark_non_differentiable(indices)
        return feats, indices

    @staticmethod
    def backward(ctx, grad, _grad_indices):
        (indices,) = ctx.saved_tensors
        shape, spatial = ctx.meta
        out = torch.empty(shape, dtype=grad.dtype, device=grad.device)
        if indices.shape[0] == 0:
            return out.zero_()
        _dense_call("spc_dense_scatter", grad.contiguous(), indices, shape[0], spatial, False, out)
        return out


def _cell_numbers(indices, spatial):
    lin = indices[:, 0].long()
    for d, s in enumerate(spatial):
        lin = lin * s + indices[:, d + 1]
    return lin


def expand_nd(ndim: int, val) -> list[int]:
    if isinstance(val, int):
        res = [val] * ndim
    else:
        res = list(val)
    if len(res) != ndim:
        raise AssertionError
    return [int(v) for v in res]
