"""Containers and thin wrappers (reference: spconv_triton/pytorch/modules.py)."""

from __future__ import annotations

import threading
import time
from collections import OrderedDict

import torch
from torch import nn

from spconv_triton_b200 import _lib

from .core import SparseConvTensor

_depth = threading.local()  # nesting depth of SparseSequential.forward on this thread


class SparseModule(nn.Module):
    """Marks a module as taking and returning SparseConvTensor."""

    def __init__(self, name=None):
        super().__init__()
        self.name = name
        self._sparse_unique_name = ""


def is_spconv_module(module):
    return isinstance(module, (SparseModule, SparseBatchNorm, SparseReLU))


def is_sparse_conv(module):
    from .conv import SparseConvolution

    return isinstance(module, SparseConvolution)


class SparseSequential(SparseModule):
    """Sequential container: sparse-aware children receive the SparseConvTensor,
    every other module is applied to its features."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        if len(args) == 1 and isinstance(args[0], OrderedDict):
            for key, module in args[0].items():
                self.add_module(key, module)
        else:
            for idx, module in enumerate(args):
                self.add_module(str(idx), module)
        for name, module in kwargs.items():
            if name in self._modules:
                raise ValueError("name exists.")
            self.add_module(name, module)

    def __len__(self):
        return len(self._modules)

    def __getitem__(self, idx):
        n = len(self)
        if not (-n <= idx < n):
            raise IndexError(f"index {idx} is out of range")
        return list(self._modules.values())[idx % n]

    def add(self, module, name=None):
        if name is None:
            name = str(len(self._modules))
            if name in self._modules:
                raise KeyError("name exists")
        self.add_module(name, module)

    def forward(self, x):
        from . import runahead

        # the outermost container of a CUDA pass looks at the status its device posted during an
        # earlier pass (raises without waiting) and posts the status of this pass when it is done
        device = None
        if isinstance(x, SparseConvTensor) and x.features.is_cuda and not getattr(_depth, "n", 0):
            device = x.features.device
            _lib.raise_posted_status(device)
        if isinstance(x, SparseConvTensor) and getattr(x, "_planner", None) is None:
            from . import sequence

            done = sequence.forward(self, x)  # the whole pass as one library call, where it applies
            if done is not None:
                if device is not None:
                    _lib.post_device_status(device)
                return done
        _depth.n = getattr(_depth, "n", 0) + 1
        entered, owned = x, runahead.begin(self, x)
        try:
            x = self._run(x)
        finally:
            _depth.n -= 1
            if owned is not None:
                owned.join_late()
                entered._planner = None
        if owned is not None and isinstance(x, SparseConvTensor):
            x._planner = None
        if device is not None and not torch.cuda.is_current_stream_capturing():
            _lib.post_device_status(device)
        return x

    def _run(self, x):
        mods = list(self._modules.values())
        i = 0
        while i < len(mods):
            module = mods[i]
            fused = _try_fold_bn_relu(mods, i, x)
            if fused is not None:
                x, i = fused
            else:
                if is_spconv_module(module):
                    x = module(x)
                elif isinstance(x, SparseConvTensor):
                    if x.indices.shape[0] != 0:
                        x = x.replace_feature(module(x.features))
                else:
                    x = module(x)
                i += 1
            # the GEMM of this layer is queued: build the next rulebook beside it
            if is_sparse_conv(module) and isinstance(x, SparseConvTensor) and x._planner is not None:
                x._planner.advance()
        return x


def _folded_bn(bn: nn.BatchNorm1d):
    """fp32 (scale, shift) with bn(x) == x * scale + shift in evaluation mode;
    memoised on the module until one of its tensors changes."""
    tensors = (bn.weight, bn.bias, bn.running_mean, bn.running_var)
    key = tuple((t._version, t.data_ptr()) if t is not None else None for t in tensors) + (bn.eps,)
    cached = getattr(bn, "_spc_folded", None)
    if cached is not None and cached[0] == key:
        return cached[1], cached[2]
    with torch.no_grad():
        scale = torch.rsqrt(bn.running_var.float() + bn.eps)
        if bn.weight is not None:
            scale = scale * bn.weight.float()
        shift = -bn.running_mean.float() * scale
        if bn.bias is not None:
            shift = shift + bn.bias.float()
        scale, shift = scale.contiguous(), shift.contiguous()
    bn._spc_folded = (key, scale, shift)
    return scale, shift


def _try_fold_bn_relu(mods, i, x):
    """In evaluation mode a sparse convolution followed by BatchNorm1d (and
    optionally ReLU) runs as ONE kernel: the normalisation becomes a per-channel
    scale and shift applied, with the ReLU, while the GEMM stores its rows.  This
    removes two passes over the activations; the result differs from the
    separate modules only by fp16 rounding order.  Switch:
    ``spconv_triton_b200.constants.SPCONV_FOLD_BN_RELU``.  Returns
    ``(new_x, next_index)`` or None when the pattern does not apply."""
    from spconv_triton_b200 import constants

    from .conv import SparseConvolution

    if not constants.SPCONV_FOLD_BN_RELU or i + 1 >= len(mods) or not isinstance(x, SparseConvTensor):
        return None
    conv, bn = mods[i], mods[i + 1]
    if not (isinstance(conv, SparseConvolution) and conv.can_fold_epilogue()):
        return None
    if not (type(bn) in (nn.BatchNorm1d, SparseBatchNorm) and not bn.training and bn.track_running_stats
            and bn.running_mean is not None and bn.num_features == conv.out_channels):
        return None
    if not x.features.is_cuda or x.features.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        return None
    if x.benchmark or x.indices.shape[0] == 0:
        return None
    relu = i + 2 < len(mods) and type(mods[i + 2]) in (nn.ReLU, SparseReLU)
    scale, shift = _folded_bn(bn)
    if scale.device != x.features.device:
        return None
    return conv(x, _fold=(scale, shift, relu)), i + 2 + int(relu)


def assign_name_for_sparse_modules(module: nn.Module):
    for k, n in module.named_modules():
        if isinstance(n, SparseModule):
            n._sparse_unique_name = k


def _on_features(base):
    """Subclass of a dense torch module that also accepts a SparseConvTensor."""

    class _Wrapped(base):
        def forward(self, x):
            if isinstance(x, SparseConvTensor):
                return x.replace_feature(super().forward(x.features))
            return super().forward(x)

    return _Wrapped


def _named(cls, name):
    cls.__name__ = cls.__qualname__ = name
    cls.__module__ = __name__
    return cls


SparseBatchNorm = _named(_on_features(nn.BatchNorm1d), "SparseBatchNorm")
SparseSyncBatchNorm = _named(_on_features(nn.SyncBatchNorm), "SparseSyncBatchNorm")
SparseReLU = _named(_on_features(nn.ReLU), "SparseReLU")
SparseIdentity = _named(_on_features(nn.Identity), "SparseIdentity")


class PrintTensorMeta(nn.Module):
    def forward(self, x):
        ft = x.features if isinstance(x, SparseConvTensor) else x
        if isinstance(ft, torch.Tensor):
            print(ft.min(), ft.max(), ft.mean())
        return x


class PrintCurrentTime(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.first_time = time.time()

    def forward(self, x, msg="", reset: bool = False):
        if reset:
            self.first_time = time.time()
        torch.cuda.synchronize()
        print(msg, time.time() - self.first_time)
        return x
