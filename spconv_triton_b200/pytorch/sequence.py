"""Inference pass of a SparseSequential through ``spc_sequence_forward`` (not in
the reference).

The reference runs a network layer by layer from Python
(spconv_triton/pytorch/modules.py:30-100).  For a VoxelNet-sized backbone on
B200 the host work of that loop (rulebook calls, dozens of small allocations,
Python between every launch) takes about twice as long as the kernels.  When a
container consists only of implicit-gemm convolutions, each optionally followed
by an evaluation-mode BatchNorm1d and a ReLU, the whole pass is handed to the
library in ONE call: it carves every table, workspace and activation out of
one arena tensor and keeps the rulebook chain ahead of the GEMMs on its own
streams.  The tensors that come back are views of that arena and are the same
ones the layer-by-layer path produces (same kernels, same arguments), rulebook
cache entries included; anything this path does not cover -- training,
autograd, Native-algorithm or inverse layers, fp32 features, pre-existing
rulebooks, benchmarking mode -- returns None and the caller runs the modules
one by one as before.  Switch: ``constants.SPCONV_NATIVE_SEQUENCE``.
"""

from __future__ import annotations

import ctypes
import functools
import threading

import numpy as np
import torch
from torch import nn

from spconv_triton_b200 import _lib, constants
from spconv_triton_b200.core import ConvAlgo

from ._impl import gemm as _gemm
from ._impl import pairs as _pairs
from .core import ImplicitGemmIndiceData, SparseConvTensor

class SeqLayer(ctypes.Structure):
    """Mirror of ``spc_seq_layer``."""

    _fields_ = [("geom", _lib.Geometry), ("rulebook", ctypes.c_int32), ("c_in", ctypes.c_int32),
                ("c_out", ctypes.c_int32), ("weight", ctypes.c_void_p), ("bias", ctypes.c_void_p),
                ("scale", ctypes.c_void_p), ("shift", ctypes.c_void_p), ("act", ctypes.c_int32),
                ("act_alpha", ctypes.c_float)]


class SeqResult(ctypes.Structure):
    """Mirror of ``spc_seq_result``."""

    _fields_ = [("n_in", ctypes.c_int64), ("n_out", ctypes.c_int64), ("workspace", ctypes.c_uint64),
                ("workspace_bytes", ctypes.c_uint64), ("out_indices", ctypes.c_uint64), ("pair_fwd", ctypes.c_uint64),
                ("pair_fwd_rowmajor", ctypes.c_uint64), ("pair_mask", ctypes.c_uint64),
                ("mask_argsort", ctypes.c_uint64), ("num_per_loc", ctypes.c_uint64), ("features", ctypes.c_uint64),
                ("masks_are_exact", ctypes.c_int64)]


class _Step:
    """One convolution of the plan with what follows it."""

    __slots__ = ("conv", "bn", "relu", "kv", "in_shape", "out_shape", "rulebook", "generates")


class _Plan:
    __slots__ = ("steps", "layers", "results", "signature", "out_shape", "bytes_per_voxel", "arena_bytes")


def _flatten(container, out) -> bool:
    from .modules import SparseSequential

    for m in container._modules.values():
        if isinstance(m, SparseSequential):
            if not _flatten(m, out):
                return False
        else:
            out.append(m)
    return True


def _compile(container, x) -> _Plan | None:
    """The plan for ``container`` applied to tensors like ``x``, or None when a
    child or a setting is outside what the native pass covers."""
    from .conv import SparseConvolution
    from .modules import SparseBatchNorm, SparseReLU

    mods: list = []
    if not _flatten(container, mods) or not mods:
        return None
    steps, i = [], 0
    shape = list(x.spatial_shape)
    keys: dict = {}
    while i < len(mods):
        conv = mods[i]
        if not isinstance(conv, SparseConvolution):
            return None
        if (conv.training or conv.conv1x1 or conv.inverse or conv.algo != ConvAlgo.MaskImplicitGemm
                or conv.record_voxel_count or conv.act_type.name != "None_" or conv.groups != 1
                or len(conv.kernel_size) != len(shape)):
            return None
        st = _Step()
        st.conv, st.bn, st.relu = conv, None, False
        st.kv = int(np.prod(conv.kernel_size))
        if not 1 < st.kv <= 32:
            return None
        if conv.subm and any(int(k) % 2 == 0 for k in conv.kernel_size):
            return None  # the layer raises its own error
        i += 1
        if i < len(mods) and type(mods[i]) in (nn.BatchNorm1d, SparseBatchNorm):
            bn = mods[i]
            if (bn.training or not bn.track_running_stats or bn.running_mean is None
                    or bn.num_features != conv.out_channels):
                return None
            st.bn = bn
            i += 1
            if i < len(mods) and type(mods[i]) in (nn.ReLU, SparseReLU):
                st.relu = True
                i += 1
        st.in_shape = list(shape)
        st.out_shape = [int(v) for v in conv._output_spatial_shape(shape)]
        if any(v <= 0 for v in st.out_shape):
            return None
        st.generates = True
        st.rulebook = len(steps)
        key = conv.indice_key
        if key is not None:
            if key in x.indice_dict:
                return None  # a rulebook made elsewhere: the module path knows how to reuse or reject it
            if key in keys:
                first = steps[keys[key]]
                same = (conv.subm and first.conv.subm and conv.kernel_size == first.conv.kernel_size
                        and conv.dilation == first.conv.dilation and first.in_shape == st.in_shape
                        and all(s.conv.subm for s in steps[keys[key]:]))
                if not same:
                    return None
                st.generates, st.rulebook = False, keys[key]
            else:
                keys[key] = len(steps)
        steps.append(st)
        shape = st.out_shape
    if not steps or len(steps) > 64:
        return None
    plan = _Plan()
    plan.steps = steps
    plan.layers = (SeqLayer * len(steps))()
    plan.results = (SeqResult * len(steps))()
    plan.out_shape = shape
    plan.bytes_per_voxel = 0.0
    plan.arena_bytes = 0
    for st, L in zip(steps, plan.layers):
        c = st.conv
        L.geom = _lib.make_geometry(x.batch_size, st.in_shape, st.out_shape, c.kernel_size, c.stride, c.padding,
                                    c.dilation, c.subm, c.transposed)
        L.rulebook, L.c_in, L.c_out = st.rulebook, c.in_channels, c.out_channels
    return plan


def _signature(container, x):
    mods: list = []
    _flatten(container, mods)
    return (tuple((id(m), m.training) for m in mods), tuple(x.spatial_shape), x.batch_size, x.indices.shape[1],
            tuple(x.indice_dict.keys()))


_ITEMSIZE = {torch.float16: 2, torch.bfloat16: 2, torch.int32: 4}
# first guess of the arena size, before a pass has told how much a plan needs
_ARENA_BYTES_PER_VOXEL = 6144.0
_ARENA_MARGIN = 64 << 20
_ARENA_GRANULE = 128 << 20


def _view(arena, offset, count, dtype, shape):
    return arena[offset:offset + count * _ITEMSIZE[dtype]].view(dtype).view(shape)


def forward(container, x):
    """Runs ``container`` on ``x`` through the native pass; None if it does not apply."""
    if not (constants.SPCONV_NATIVE_SEQUENCE and constants.SPCONV_FOLD_BN_RELU and constants.SPCONV_RULEBOOK_RUNAHEAD):
        return None
    if torch.is_grad_enabled() or not isinstance(x, SparseConvTensor) or x.benchmark:
        return None
    feats, indices = x.features, x.indices
    if (not feats.is_cuda or feats.dtype not in (torch.float16, torch.bfloat16) or indices.shape[0] == 0
            or indices.dtype != torch.int32 or _gemm.GEMM_PATH != _lib.SPC_GEMM_AUTO
            or torch.cuda.is_current_stream_capturing()):
        return None
    # one plan per host thread: its layer and result arrays are written during a pass, and passes
    # may run concurrently from several threads (parallel.PassPipeline)
    sig = _signature(container, x)
    plans = container.__dict__.setdefault("_spc_plans", {})
    me = threading.get_ident()
    cached = plans.get(me)
    if cached is None or cached.signature != sig:
        plan = _compile(container, x)
        if plan is None:
            plans.pop(me, None)
            return None
        plan.signature = sig
        plans[me] = plan
    else:
        plan = cached
    steps = plan.steps
    if steps[0].conv.in_channels != feats.shape[1]:
        return None
    dev = feats.device
    from .modules import _folded_bn
    from .runahead import _side_stream

    # pointers of this pass (weights and folded statistics may have changed since the last one)
    keep = []
    for st, L in zip(steps, plan.layers):
        c = st.conv
        w = c.weight
        if w.dtype != feats.dtype or w.device != dev or not w.is_contiguous():
            return None
        L.weight = w.data_ptr()
        b = c.bias
        if b is not None and (b.dtype != feats.dtype or b.device != dev):
            return None
        L.bias = b.data_ptr() if b is not None else None
        if st.bn is not None:
            scale, shift = _folded_bn(st.bn)
            if scale.device != dev:
                return None
            keep += [scale, shift]
            L.scale, L.shift = scale.data_ptr(), shift.data_ptr()
        else:
            L.scale = L.shift = None
        L.act = _lib.SPC_ACT_RELU if st.relu else _lib.SPC_ACT_NONE
        L.act_alpha = 0.0

    feats = feats.contiguous()
    indices = indices.contiguous()
    n_in = int(indices.shape[0])
    lib = _lib.load()
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        chain, side = _side_stream(dev, 0), _side_stream(dev, 1)
        # sized from the largest need per input voxel seen so far and rounded up coarsely, so that
        # passes over scenes of similar size ask the caching allocator for the same block again
        # [bytes, bytes per voxel] shared by the plans of all host threads: a thread that meets
        # its largest scene late would otherwise grow its arena (one cudaMalloc, which
        # synchronises the device) long after the others have
        floor = container.__dict__.setdefault("_spc_arena_floor", [0, 0.0])
        per_voxel = max(plan.bytes_per_voxel, floor[1]) or _ARENA_BYTES_PER_VOXEL
        arena_bytes = int(per_voxel * n_in * 1.2) + _ARENA_MARGIN
        arena_bytes = -(-arena_bytes // _ARENA_GRANULE) * _ARENA_GRANULE
        # never smaller than the last one: equal requests are what the caching allocator serves
        # from its free list without splitting or growing
        arena_bytes = plan.arena_bytes = floor[0] = max(arena_bytes, plan.arena_bytes, floor[0])
        needed = ctypes.c_size_t(0)
        for _attempt in range(4):
            # The rulebook streams touch the arena and the indices only inside the call, and the
            # caller's stream joins both before the call returns: to the caching allocator the
            # arena is a block of the caller's stream like any other (no record_stream, whose
            # deferred frees made the pool grow in bursts when several threads run passes).
            arena = torch.empty(arena_bytes, dtype=torch.uint8, device=dev)
            rc = lib.spc_sequence_forward(ctypes.cast(plan.layers, ctypes.c_void_p), len(steps), indices.data_ptr(),
                                          feats.data_ptr(), n_in, _lib.dtype_code(feats.dtype), arena.data_ptr(),
                                          arena_bytes, ctypes.cast(ctypes.pointer(needed), ctypes.c_void_p),
                                          ctypes.cast(plan.results, ctypes.c_void_p), main.cuda_stream,
                                          chain.cuda_stream, side.cuda_stream)
            if rc == _lib.SPC_OK:
                break
            # whatever was queued wrote into this arena: let it finish before the arena goes away
            main.synchronize()
            chain.synchronize()
            side.synchronize()
            if rc != _lib.SPC_ERR_WORKSPACE_TOO_SMALL:
                return None  # e.g. a layer without output points: the modules raise the proper error
            arena_bytes = int(needed.value * 1.5) + _ARENA_MARGIN
            arena_bytes = plan.arena_bytes = floor[0] = -(-arena_bytes // _ARENA_GRANULE) * _ARENA_GRANULE
        else:
            return None
        plan.bytes_per_voxel = floor[1] = max(plan.bytes_per_voxel, floor[1], needed.value / n_in)
        return _wrap(plan, x, indices, arena, dev, keep)


_ABSENT = 0xFFFFFFFFFFFFFFFF  # offset of a table the pass did not produce


def _column_major(rowmajor, kv, late, table=None):
    """The [kv, n_out] table with the attributes the operator layer looks for on it; transposed out
    of the row-major copy when the pass did not write it."""
    if table is None:
        table = rowmajor[:, :kv].t().contiguous()
    table._spc_rowmajor = rowmajor
    if late is not None:
        table._spc_late = late
    return table


def _exact_masks(rowmajor, kv):
    """``pair_mask_fwd_splits`` / ``mask_argsort_fwd_splits`` as the rulebook generator emits them (one
    split): the rows' mask words sorted ascending, stable, and their argsort.  The pass itself orders
    the rows by a different key (rows that share kernel offsets end up in the same GEMM tile), so
    these two are made from the row-major table when somebody reads them."""
    weights = torch.ones(kv, dtype=torch.int64, device=rowmajor.device) << torch.arange(kv, device=rowmajor.device)
    words = ((rowmajor[:, :kv] >= 0).to(torch.int64) * weights).sum(1)
    vals, args = torch.sort(words, stable=True)
    vals = torch.where(vals >= 2 ** 31, vals - 2 ** 32, vals)  # the words are unsigned, the tensor is int32
    return [vals.to(torch.int32).reshape(-1, 1)], [args.to(torch.int32)]


def _wrap(plan, x, indices, arena, dev, keep):
    """The output tensor and the rulebook cache entries, as views of the arena."""
    steps, results = plan.steps, plan.results
    ndim = len(x.spatial_shape)
    indice_dict = dict(x.indice_dict)
    cur_indices, masks = indices, None
    for st, L, R in zip(steps, plan.layers, results):
        if not st.generates:
            continue
        c, kv, kvp = st.conv, st.kv, (st.kv + 3) // 4 * 4
        n_in, n_out = int(R.n_in), int(R.n_out)
        in_indices = cur_indices
        if not c.subm:
            cur_indices = _view(arena, R.out_indices, n_out * (ndim + 1), torch.int32, (n_out, ndim + 1))
        if c.indice_key is None:
            continue
        rowmajor = _view(arena, R.pair_fwd_rowmajor, n_out * kvp, torch.int32, (n_out, kvp))
        late = None
        if not c.subm:
            # the input-side tables stay pending; they are built from the workspace when somebody reads them
            p = _pairs._Prepared()
            p.geom, p.indices, p.n_in, p.n_out, p.out_shape, p.kv, p.subm = L.geom, in_indices, n_in, n_out, st.out_shape, kv, False
            p.workspace = arena[R.workspace:R.workspace + R.workspace_bytes]
            late = _pairs.LateTables(p, n_out, (ctypes.c_uint32 * 1)(0xFFFFFFFF), 1, True, 1)
        if R.pair_fwd != _ABSENT:
            pair_fwd = _column_major(rowmajor, kv, late, _view(arena, R.pair_fwd, kv * n_out, torch.int32, (kv, n_out)))
        else:
            pair_fwd = None  # not written: no layer of the pass reads it
        exact = int(R.masks_are_exact) != 0
        pm = [_view(arena, R.pair_mask, n_out, torch.int32, (n_out, 1))] if exact else None
        ma = [_view(arena, R.mask_argsort, n_out, torch.int32, (n_out,))] if exact else None
        masks = [np.array([0xFFFFFFFF], dtype=np.uint32)]
        data = ImplicitGemmIndiceData(
            in_indices if c.subm else cur_indices, in_indices, pair_fwd, torch.Tensor(), pm, [], ma, [], masks,
            st.in_shape, st.out_shape, c.subm, c.algo, c.kernel_size, c.stride, c.dilation, c.padding)
        if not exact:
            data._masks_fwd_thunk = functools.partial(_exact_masks, rowmajor, kv)
        if pair_fwd is None:
            data._pair_fwd_thunk = functools.partial(_column_major, rowmajor, kv, late)
        data._late = late
        indice_dict[c.indice_key] = data
    last, R = steps[-1], results[len(steps) - 1]
    feats = _view(arena, R.features, int(R.n_out) * last.conv.out_channels, x.features.dtype,
                  (int(R.n_out), last.conv.out_channels))
    out = SparseConvTensor(feats, cur_indices, plan.out_shape, x.batch_size, x.grid, x.voxel_num, indice_dict)
    x._carry_over(out)
    out._planner = None
    out._spc_keep = keep  # folded statistics in use by kernels that may still be queued
    return out
