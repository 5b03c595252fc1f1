"""Sparse max / average pooling layers (reference: spconv_triton/pytorch/pool.py)."""

from __future__ import annotations

import time as _time

import numpy as np
import torch

from spconv_triton_b200.core import ConvAlgo

from . import functional as Fsp
from . import ops
from .conv import _MAX_NUM_VOXELS_DURING_TRAINING
from .core import IndiceData, SparseConvTensor, expand_nd, register_implicit_gemm_indice_data
from .modules import SparseModule

CPU_ONLY_BUILD = False


class _SparsePoolBase(SparseModule):
    """Geometry handling shared by max and average pooling."""

    def _setup(self, ndim, kernel_size, stride, padding, dilation, indice_key, subm, record_voxel_count):
        self.ndim = ndim
        self.kernel_size = expand_nd(ndim, kernel_size)
        # stride=None means "same as the kernel"
        self.stride = self.kernel_size.copy() if stride is None else expand_nd(ndim, stride)
        self.padding = expand_nd(ndim, padding)
        self.subm = subm
        if record_voxel_count and not subm:
            self.register_buffer(_MAX_NUM_VOXELS_DURING_TRAINING, torch.zeros(1, dtype=torch.int32))
        self.record_voxel_count = record_voxel_count
        self.dilation = expand_nd(ndim, dilation)
        self.indice_key = indice_key
        return int(np.prod(kernel_size))

    def extra_repr(self):
        parts = [f"kernel_size={self.kernel_size}, stride={self.stride}"]
        if self.padding != (0,) * len(self.padding):
            parts.append(f"padding={self.padding}")
        if self.dilation != (1,) * len(self.dilation):
            parts.append(f"dilation={self.dilation}")
        if self.algo is not None:
            parts.append(f"algo={self.algo}")
        return ", ".join(parts)

    def get_max_num_voxels(self) -> torch.Tensor | None:
        return getattr(self, _MAX_NUM_VOXELS_DURING_TRAINING, None)

    def _out_shape(self, spatial_shape):
        if self.subm:
            return spatial_shape
        return ops.get_conv_output_size(spatial_shape, self.kernel_size, self.stride, self.padding,
                                        self.dilation)

    def _igemm_tables(self, x, indice_dict, out_spatial_shape):
        res = ops.get_indice_pairs_implicit_gemm(
            x.indices, x.batch_size, x.spatial_shape, self.algo, ksize=self.kernel_size, stride=self.stride,
            padding=self.padding, dilation=self.dilation, out_padding=[0] * self.ndim, subm=self.subm,
            is_train=(not self.subm) or self.training, alloc=x.thrust_allocator, timer=x._timer)
        if self.indice_key is not None:
            register_implicit_gemm_indice_data(
                indice_dict, self.indice_key, res, x.indices, is_subm=self.subm,
                spatial_shape=x.spatial_shape, out_spatial_shape=out_spatial_shape, algo=self.algo,
                ksize=self.kernel_size, stride=self.stride, dilation=self.dilation, padding=self.padding)
        return res[0], res[2], res[3]

    def _finish(self, x, out_tensor, out_features, outids, indice_dict, out_spatial_shape):
        if not self.subm and self.record_voxel_count and hasattr(self, _MAX_NUM_VOXELS_DURING_TRAINING):
            ops.maximum_value_int_(getattr(self, _MAX_NUM_VOXELS_DURING_TRAINING), outids.shape[0])
        out_tensor = out_tensor.replace_feature(out_features)
        out_tensor.indices = outids
        out_tensor.indice_dict = indice_dict
        out_tensor.spatial_shape = out_spatial_shape
        return out_tensor


class SparseMaxPool(_SparsePoolBase):
    def __init__(self, ndim, kernel_size=3, stride=1, padding=0, dilation=1, indice_key: str | None = None,
                 subm: bool = False, algo: ConvAlgo | None = None, record_voxel_count: bool = False,
                 name=None):
        super().__init__(name=name)
        kv = self._setup(ndim, kernel_size, stride, padding, dilation, indice_key, subm, record_voxel_count)
        if algo is None:
            algo = ConvAlgo.MaskImplicitGemm if kv <= 128 else ConvAlgo.Native
        if kv > 128 and algo != ConvAlgo.Native:
            raise AssertionError("implicit gemm don't support kv >= 32 for now")
        self.algo = algo

    @torch.compiler.disable
    def forward(self, x: SparseConvTensor):
        if x.is_quantized:
            raise NotImplementedError("int8 is not supported by spconv_triton")
        if not isinstance(x, SparseConvTensor):
            raise AssertionError
        features = x.features
        out_spatial_shape = self._out_shape(x.spatial_shape)
        out_tensor = x.shadow_copy()
        if x.benchmark:
            if self.name is None:
                raise ValueError("you need to assign name to spmodules before benchmark "
                                 "(spconv.utils.bench.assign_name_to_spmod)")
            x.benchmark_record.setdefault(self.name, {
                "type": "SparseMaxPool", "indice_gen_time": [], "time": [], "num_points": [],
                "num_out_points": [],
                "params": {"kernel_size": self.kernel_size, "stride": self.stride, "padding": self.padding,
                           "dilation": self.dilation, "channels": features.shape[1]},
            })
            torch.cuda.synchronize()
            t0 = _time.time()
        indice_dict = x.indice_dict.copy()
        if self.algo == ConvAlgo.Native:
            outids, pairs, pair_num = ops.get_indice_pairs(
                x.indices, x.batch_size, x.spatial_shape, ConvAlgo.Native, self.kernel_size, self.stride,
                self.padding, self.dilation, [0] * self.ndim, False)
            if x.benchmark:
                # for the Native path the recorded kernel time excludes rulebook generation
                torch.cuda.synchronize()
                out_tensor.benchmark_record[self.name]["indice_gen_time"].append(_time.time() - t0)
                t0 = _time.time()
            if self.indice_key is not None:
                if x.find_indice_pair(self.indice_key) is not None:
                    raise ValueError(f"indice key {self.indice_key} exists")
                indice_dict[self.indice_key] = IndiceData(
                    outids, x.indices, pairs, pair_num, x.spatial_shape, out_spatial_shape, is_subm=False,
                    algo=self.algo, ksize=self.kernel_size, stride=self.stride, padding=self.padding,
                    dilation=self.dilation)
            out_features = Fsp.indice_maxpool(features, pairs.to(features.device),
                                              pair_num.to(features.device), outids.shape[0])
        else:
            outids, pair_fwd, pair_bwd = self._igemm_tables(x, indice_dict, out_spatial_shape)
            out_features = Fsp.indice_maxpool_implicit_gemm(features, pair_fwd, pair_bwd, outids.shape[0])
        if x.benchmark:
            torch.cuda.synchronize()
            rec = out_tensor.benchmark_record[self.name]
            rec["time"].append(_time.time() - t0)
            rec["num_points"].append(features.shape[0])
            rec["num_out_points"].append(out_features.shape[0])
        return self._finish(x, out_tensor, out_features, outids, indice_dict, out_spatial_shape)


class SparseAvgPool(_SparsePoolBase):
    """Average over the inputs that are present in each window."""

    def __init__(self, ndim, kernel_size=3, stride=1, padding=0, dilation=1, indice_key: str | None = None,
                 subm: bool = False, algo: ConvAlgo | None = None, record_voxel_count: bool = False,
                 name=None):
        super().__init__(name=name)
        kv = self._setup(ndim, kernel_size, stride, padding, dilation, indice_key, subm, record_voxel_count)
        if kv > 32:
            raise AssertionError("avg pool only support implicit-gemm style indice gen with kv <= 32 limit")
        self.algo = ConvAlgo.MaskImplicitGemm

    @torch.compiler.disable
    def forward(self, x):
        if x.is_quantized:
            raise NotImplementedError("int8 is not supported by spconv_triton")
        if not isinstance(x, SparseConvTensor):
            raise AssertionError
        out_spatial_shape = self._out_shape(x.spatial_shape)
        out_tensor = x.shadow_copy()
        indice_dict = x.indice_dict.copy()
        outids, pair_fwd, pair_bwd = self._igemm_tables(x, indice_dict, out_spatial_shape)
        out_features = Fsp.indice_avgpool_implicit_gemm(x.features, pair_fwd, pair_bwd, outids.shape[0],
                                                        self.training)
        return self._finish(x, out_tensor, out_features, outids, indice_dict, out_spatial_shape)


class SparseGlobalMaxOrAvgPool(SparseModule):
    """Per-sample reduction over all points.  The average variant returns
    channel 0 of the mean only (shape [batch]), as upstream does."""

    def __init__(self, is_mean: bool, name=None):
        super().__init__(name=name)
        self.is_mean = is_mean

    @torch.compiler.disable
    def forward(self, x: SparseConvTensor):
        if x.is_quantized:
            raise NotImplementedError("int8 is not supported by spconv_triton")
        if not isinstance(x, SparseConvTensor):
            raise AssertionError
        if not x.features.is_cuda:
            raise NotImplementedError("spconv_triton_b200 global pooling is CUDA only")
        return _GlobalPool.apply(x.features, x.indices, int(x.batch_size), bool(self.is_mean))


class _GlobalPool(torch.autograd.Function):
    """One pass of ``spc_global_pool`` over the features; the gradient goes to the row that held
    each maximum, or evenly to channel 0 of a sample's rows for the mean."""

    @staticmethod
    def forward(ctx, features, indices, batch_size, is_mean):
        from spconv_triton_b200 import _lib

        features, indices = features.contiguous(), indices.contiguous()
        n, c = int(features.shape[0]), int(features.shape[1])
        dev = features.device
        lib = _lib.load()
        out = torch.empty([batch_size] if is_mean else [batch_size, c], dtype=features.dtype, device=dev)
        argmax = None if is_mean else torch.empty([batch_size, c], dtype=torch.int32, device=dev)
        counts = torch.empty([batch_size], dtype=torch.int32, device=dev)
        ws = torch.empty(lib.spc_global_pool_workspace_bytes(batch_size, c), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.spc_global_pool(
                _lib.ptr(features), _lib.ptr(indices), n, c, int(indices.shape[1]), batch_size,
                _lib.dtype_code(features.dtype), int(is_mean), _lib.ptr(ws), ws.numel(), _lib.ptr(out),
                _lib.ptr(argmax), _lib.ptr(counts), _lib.current_stream(dev)))
        if not is_mean and bool((counts == 0).any()):
            # torch.max over zero rows raises in the reference as well (pool.py:262)
            raise RuntimeError("SparseGlobalMaxPool: a sample has no voxels")
        if is_mean:
            ctx.save_for_backward(indices, counts)
        else:
            ctx.save_for_backward(argmax)
        ctx.meta = (n, c, is_mean)
        return out

    @staticmethod
    def backward(ctx, grad):
        n, c, is_mean = ctx.meta
        gin = torch.zeros([n, c], dtype=grad.dtype, device=grad.device)
        if is_mean:
            indices, counts = ctx.saved_tensors
            gin[:, 0] = (grad / counts.to(grad.dtype))[indices[:, 0].long()]
        else:
            (argmax,) = ctx.saved_tensors
            cols = torch.arange(c, device=grad.device).expand_as(argmax)
            gin[argmax.long().reshape(-1), cols.reshape(-1)] = grad.reshape(-1)
        return gin, None, None, None


class SparseGlobalAvgPool(SparseGlobalMaxOrAvgPool):
    def __init__(self, name=None):
        super().__init__(is_mean=True, name=name)


class SparseGlobalMaxPool(SparseGlobalMaxOrAvgPool):
    def __init__(self, name=None):
        super().__init__(is_mean=False, name=name)


def _leaf(name, base, ndim):
    class Leaf(base):
        def __init__(self, kernel_size, stride=None, padding=0, dilation=1, indice_key=None,
                     algo: ConvAlgo | None = None, record_voxel_count: bool = False, name=None):
            super().__init__(ndim, kernel_size, stride, padding, dilation, indice_key=indice_key, algo=algo,
                             record_voxel_count=record_voxel_count, name=name)

    Leaf.__name__ = Leaf.__qualname__ = name
    Leaf.__module__ = __name__
    Leaf.__doc__ = base.__doc__
    return Leaf


SparseMaxPool1d, SparseMaxPool2d, SparseMaxPool3d, SparseMaxPool4d = (
    _leaf(f"SparseMaxPool{d}d", SparseMaxPool, d) for d in (1, 2, 3, 4))
SparseAvgPool1d, SparseAvgPool2d, SparseAvgPool3d = (
    _leaf(f"SparseAvgPool{d}d", SparseAvgPool, d) for d in (1, 2, 3))

ALL_POOL_LAYERS = {SparseAvgPool3d, SparseAvgPool2d, SparseAvgPool1d, SparseMaxPool1d, SparseMaxPool2d,
                   SparseMaxPool3d, SparseMaxPool4d, SparseAvgPool, SparseMaxPool}
