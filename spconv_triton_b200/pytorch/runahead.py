"""Rulebook run-ahead for SparseSequential (not in the reference).

A rulebook depends only on the voxel indices that enter its layer, never on
features, and the indices that leave layer i are part of rulebook i.  So the
whole chain rulebook 1 -> 2 -> ... can be generated independently of the
GEMMs.  SparseSequential uses that: while the gather-GEMM of layer i runs on
the caller's stream, the rulebook of the next generating layer is built on a
second, high-priority stream; the layer that consumes it makes the caller's
stream wait on the rulebook's event.  The forward time becomes about
max(rulebook chain, GEMM chain) instead of their sum.  Results are identical:
the same C-ABI calls with the same arguments, only on another stream.

The plan is conservative.  It covers SparseConvolution layers that use the
implicit-gemm rulebook inside (nested) SparseSequential containers; the first
child it cannot predict (pooling, user-defined sparse modules, the Native
algorithm) ends the look-ahead and everything after runs inline as before.  A
planned rulebook is only used when the layer is called with exactly the index
tensor it was generated from; anything raised while planning is dropped so that
the layer raises it itself, at its own place.
Switch: ``spconv_triton_b200.constants.SPCONV_RULEBOOK_RUNAHEAD``.
"""

from __future__ import annotations

import threading

import torch

from spconv_triton_b200.core import ConvAlgo

from .. import constants
from . import ops
from ._impl import pairs as _pairs
from .core import ImplicitGemmIndiceData, SparseConvTensor, register_implicit_gemm_indice_data

_side_streams: dict = {}


def _side_stream(device: torch.device, which: int) -> torch.cuda.Stream:
    # one set per host thread: passes issued from different threads must not queue behind (or
    # synchronise on) each other's rulebook work
    key = (device.index if device.index is not None else torch.cuda.current_device(), which, threading.get_ident())
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device, priority=-1)
    return _side_streams[key]


def _tensors_of(res):
    """Every tensor a rulebook tuple holds, with the row-major table copies."""
    stack = [res]
    while stack:
        item = stack.pop()
        if isinstance(item, torch.Tensor):
            yield item
            extra = getattr(item, "_spc_rowmajor", None)
            if extra is not None:
                yield extra
        elif isinstance(item, (list, tuple)):
            stack.extend(item)


def flatten_convs(container) -> list:
    """The sparse convolutions of ``container`` in execution order, up to the
    first child whose effect on the indices cannot be predicted."""
    from .conv import SparseConvolution
    from .modules import SparseBatchNorm, SparseModule, SparseReLU, SparseSequential

    out: list = []

    def walk(seq) -> bool:
        for m in seq._modules.values():
            if isinstance(m, SparseSequential):
                if not walk(m):
                    return False
            elif isinstance(m, SparseConvolution):
                out.append(m)
            elif isinstance(m, (SparseBatchNorm, SparseReLU)):
                continue
            elif isinstance(m, SparseModule):
                return False
        return True

    walk(container)
    return out


class RulebookPlanner:
    def __init__(self, convs: list, x: SparseConvTensor):
        device = x.indices.device
        self.queue = convs
        self.pos = 0
        self.ready: dict = {}
        self.indices = x.indices
        self.spatial_shape = list(x.spatial_shape)
        self.batch_size = x.batch_size
        self.keys = dict(x.indice_dict)
        self.allocator = x.thrust_allocator
        self.timer = x._timer
        self.main = torch.cuda.current_stream(device)
        self.side = _side_stream(device, 0)
        # input-side tables of strided layers: needed by inverse layers and the backward
        # pass only, so they are built on a third stream, off the chain of rulebooks
        self.late = _pairs.DeferredBackward(_side_stream(device, 1))
        self.side.wait_stream(self.main)
        x.indices.record_stream(self.side)

    # -- planning ---------------------------------------------------------------------------
    def advance(self) -> None:
        """Keeps one generated rulebook ahead of the layer that runs now."""
        while not self.ready and self.pos < len(self.queue):
            conv = self.queue[self.pos]
            self.pos += 1
            try:
                ok = self._plan(conv)
            except Exception:
                ok = False
            if not ok:
                self.pos = len(self.queue)

    def _plan(self, conv) -> bool:
        out_shape = conv._output_spatial_shape(self.spatial_shape)
        if conv.conv1x1:
            self.spatial_shape = out_shape
            return True
        if conv.algo == ConvAlgo.Native:
            return False
        datas = self.keys.get(conv.indice_key) if conv.indice_key is not None else None
        if datas is not None and not isinstance(datas, ImplicitGemmIndiceData):
            return False
        if conv.inverse:
            if datas is None:
                return False
            self.indices, self.spatial_shape = datas.indices, list(datas.spatial_shape)
            return True
        if datas is not None:
            if not conv.subm:
                return False
            self.indices, self.spatial_shape = datas.out_indices, out_shape
            return True
        src = self.indices
        # training: the input-side tables go to the third stream; inference: they stay pending
        with torch.cuda.stream(self.side), _pairs.deferred_backward(self.late if conv.training else "late"):
            res = ops.get_indice_pairs_implicit_gemm(
                src, self.batch_size, self.spatial_shape, conv.algo, ksize=conv.kernel_size,
                stride=conv.stride, padding=conv.padding, dilation=conv.dilation,
                out_padding=conv.output_padding, subm=conv.subm, transpose=conv.transposed,
                is_train=(not conv.subm) or conv.training, alloc=self.allocator, timer=self.timer)
            event = torch.cuda.Event()
            event.record(self.side)
        self.ready[id(conv)] = (res, event, src, list(self.spatial_shape))
        if conv.indice_key is not None:
            register_implicit_gemm_indice_data(
                self.keys, conv.indice_key, res, src, is_subm=conv.subm, spatial_shape=self.spatial_shape,
                out_spatial_shape=out_shape, algo=conv.algo, ksize=conv.kernel_size, stride=conv.stride,
                dilation=conv.dilation, padding=conv.padding)
        self.indices, self.spatial_shape = res[0], out_shape
        return True

    # -- consumption ------------------------------------------------------------------------
    def take(self, conv, x: SparseConvTensor):
        """The planned rulebook of ``conv`` if it was made from exactly ``x``'s
        indices; the caller's stream is made to wait for it."""
        entry = self.ready.pop(id(conv), None)
        if entry is None:
            return None
        res, event, src, shape = entry
        if src is not x.indices or shape != list(x.spatial_shape) or x.batch_size != self.batch_size:
            self.pos = len(self.queue)  # the data flow left the plan
            return None
        main = torch.cuda.current_stream(x.indices.device)
        main.wait_event(event)
        for t in _tensors_of(res):
            if t.is_cuda:
                t.record_stream(main)
        return res


    def join_late(self) -> None:
        """Makes the caller's stream wait for every input-side table built so far."""
        if not self.late.pending:
            return
        main = torch.cuda.current_stream(self.indices.device)
        for event, tensors in self.late.pending:
            main.wait_event(event)
            for t in tensors:
                t.record_stream(main)
        self.late.pending.clear()


def begin(container, x):
    """Attaches a planner to ``x`` when ``container`` is the outermost
    SparseSequential of a CUDA forward; returns the planner it created."""
    if not constants.SPCONV_RULEBOOK_RUNAHEAD or not isinstance(x, SparseConvTensor):
        return None
    if getattr(x, "_planner", None) is not None or not x.indices.is_cuda or x.benchmark:
        return None
    if x.indices.shape[0] == 0 or torch.cuda.is_current_stream_capturing():
        return None
    convs = flatten_convs(container)
    if len(convs) < 2:
        return None
    planner = RulebookPlanner(convs, x)
    x._planner = planner
    planner.advance()
    return planner
