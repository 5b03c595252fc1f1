"""Containers and thin wrappers (reference: spconv_triton/pytorch/modules.py)."""

from __future__ import annotations

import time
from collections import OrderedDict

import torch
from torch import nn

from .core import SparseConvTensor


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
        for module in self._modules.values():
            if is_spconv_module(module):
                x = module(x)
            elif isinstance(x, SparseConvTensor):
                if x.indices.shape[0] != 0:
                    x = x.replace_feature(module(x.features))
            else:
                x = module(x)
        return x


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
