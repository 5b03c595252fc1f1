"""Rulebook generation through the C ABI.

Function names, argument order, return values and host-side errors mirror the
reference module these wrappers stand in for
(spconv_triton/pytorch/_impl/pairs.py in the reference project); the work is
done by ``spc_rulebook_*`` in libspconv_b200.so.
"""

from __future__ import annotations

import contextlib
import ctypes
import threading
import functools

import numpy as np
import torch

from spconv_triton_b200 import _lib

_POINT_VANISH_MSG = (
    "Your points vanished here, this usually happens when you provide "
    "conv params that may ignore some input points. Example: "
    "spatial_shape={}, ksize={}, stride={}, padding={}, dilation={}"
)


def _i32_array(vals):
    vals = [int(v) for v in vals]
    return (ctypes.c_int32 * len(vals))(*vals)


def get_conv_output_size(input_size, kernel_size, stride, padding, dilation):
    """Reference: _impl/pairs.py:59-70."""
    n = len(input_size)
    out = (ctypes.c_int32 * n)()
    _lib.check(_lib.load().spc_conv_output_size(n, _i32_array(input_size), _i32_array(kernel_size),
                                                _i32_array(stride), _i32_array(padding),
                                                _i32_array(dilation), out))
    return [int(v) for v in out]


def get_deconv_output_size(input_size, kernel_size, stride, padding, dilation, output_padding):
    """Reference: _impl/pairs.py:73-88."""
    n = len(input_size)
    if any(int(k) == -1 for k in kernel_size):
        raise ValueError("deconv don't support kernel_size < 0")
    out = (ctypes.c_int32 * n)()
    _lib.check(_lib.load().spc_deconv_output_size(n, _i32_array(input_size), _i32_array(kernel_size),
                                                  _i32_array(stride), _i32_array(padding),
                                                  _i32_array(dilation), _i32_array(output_padding), out))
    return [int(v) for v in out]


class _Prepared:
    """State between phase 1 (count) and phase 2 (fill) of one rulebook."""

    __slots__ = ("geom", "indices", "n_in", "n_out", "out_shape", "kv", "workspace", "subm")


def _prepare(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
             transpose) -> _Prepared:
    """Validation (same exceptions as the reference's compute_candidates,
    _impl/pairs.py:138-164,210-213) followed by ``spc_rulebook_prepare``."""
    ndim = len(spatial_shape)
    n_in = int(indices.shape[0])
    kv = int(functools.reduce(lambda a, b: a * b, [int(k) for k in ksize], 1))
    if n_in == 0:
        raise ValueError("N > 0 assert: sparse tensor has no points")
    if any(int(k) <= 0 for k in ksize):
        raise ValueError(f"kernel size {list(ksize)} not supported by pair gen")
    if subm:
        if any(int(k) % 2 == 0 for k in ksize):
            raise NotImplementedError("subm convolution requires odd kernel sizes")
        out_shape = [int(s) for s in spatial_shape]
    elif transpose:
        out_shape = get_deconv_output_size(spatial_shape, ksize, stride, padding, dilation, out_padding)
    else:
        out_shape = get_conv_output_size(spatial_shape, ksize, stride, padding, dilation)
    if any(x <= 0 for x in out_shape):
        raise ValueError(f"your out spatial shape {out_shape} reach zero!!! input shape: {list(spatial_shape)}")
    if ndim > _lib.SPC_MAX_NDIM:
        raise NotImplementedError(f"ndim {ndim} > {_lib.SPC_MAX_NDIM}")
    if indices.dtype != torch.int32:
        indices = indices.to(torch.int32)
    if not indices.is_contiguous():
        indices = indices.contiguous()

    lib = _lib.load()
    p = _Prepared()
    p.geom = _lib.make_geometry(batch_size, spatial_shape, out_shape, ksize, stride, padding, dilation, subm,
                                transpose)
    p.indices, p.n_in, p.out_shape, p.kv, p.subm = indices, n_in, out_shape, kv, bool(subm)
    nbytes = int(lib.spc_rulebook_workspace_bytes(ctypes.byref(p.geom), n_in))
    if nbytes == 0:
        raise ValueError("rulebook geometry rejected by libspconv_b200")
    with torch.cuda.device(indices.device):
        p.workspace = torch.empty(nbytes, dtype=torch.uint8, device=indices.device)
        n_out = ctypes.c_int64(0)
        _lib.check(lib.spc_rulebook_prepare(ctypes.byref(p.geom), _lib.ptr(indices), n_in,
                                            _lib.ptr(p.workspace), nbytes, ctypes.byref(n_out),
                                            _lib.current_stream(indices.device)))
    p.n_out = int(n_out.value)
    if p.n_out == 0:
        raise ValueError(_POINT_VANISH_MSG.format(list(spatial_shape), list(ksize), list(stride),
                                                  list(padding), list(dilation)))
    return p


def native_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                 transpose):
    """Reference: native_pairs, _impl/pairs.py:242-278.  Returns
    ``(out_inds, pair [2, kv, N] int32, indice_num_per_loc [kv] int32)``."""
    p = _prepare(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                 transpose)
    dev = p.indices.device
    ndim = len(spatial_shape)
    with torch.cuda.device(dev):
        out_inds = indices if subm else torch.empty((p.n_out, ndim + 1), dtype=torch.int32, device=dev)
        pair = torch.empty((2, p.kv, p.n_in), dtype=torch.int32, device=dev)
        npl = torch.empty((p.kv,), dtype=torch.int32, device=dev)
        _lib.check(_lib.load().spc_rulebook_native(
            ctypes.byref(p.geom), _lib.ptr(p.indices), p.n_in, p.n_out, _lib.ptr(p.workspace),
            p.workspace.numel(), None if subm else _lib.ptr(out_inds), _lib.ptr(pair), _lib.ptr(npl),
            _lib.current_stream(dev)))
    return out_inds, pair, npl


def _split_masks(kv, is_mask_split):
    """Reference: _impl/pairs.py:344-352."""
    if is_mask_split:
        half = kv // 2
        remain = kv - half
        one = np.array([1], dtype=np.uint64)
        first = (one << np.uint64(remain)) - np.uint64(1)
        second = ((one << np.uint64(half)) - np.uint64(1)) << np.uint64(remain)
        return [first.astype(np.uint32), second.astype(np.uint32)]
    return [np.array([0xFFFFFFFF], dtype=np.uint32)]


class DeferredBackward:
    """While one of these is installed (``deferred_backward``), igemm_pairs builds
    the input-side tables of strided layers on ``stream`` instead of the current
    one, after the forward tables, and appends ``(event, tensors)`` to
    ``pending``: whoever reads those tensors on another stream waits for the
    event first.  Used by the rulebook run-ahead of SparseSequential."""

    def __init__(self, stream):
        self.stream = stream
        self.pending: list = []


class LateTables:
    """The input-side tables of a strided layer (pair_bwd, its masks and argsort),
    not built yet.  An inference forward never reads them; an inverse layer that
    reuses the rulebook, or anyone reading them from the indice_dict entry, calls
    ``get()`` and they are built then, from the hash table the forward half left
    in the workspace."""

    def __init__(self, prepared, n_out, split_words, n_split, do_sort, mic):
        self.p, self.n_out, self.split_words, self.n_split = prepared, n_out, split_words, n_split
        self.do_sort, self.mic = do_sort, mic
        self.value = None

    def get(self):
        if self.value is None:
            p, dev = self.p, self.p.indices.device
            kv, kvp = p.kv, (p.kv + 3) // 4 * 4
            with torch.cuda.device(dev):
                stream = torch.cuda.current_stream(dev)
                for t in (p.workspace, p.indices):
                    t.record_stream(stream)
                pair_bwd = torch.empty((kv, p.n_in), dtype=torch.int32, device=dev)
                pm_bwd = torch.empty((self.n_split, p.n_in, self.mic), dtype=torch.int32, device=dev)
                ma_bwd = torch.empty((self.n_split, p.n_in), dtype=torch.int32, device=dev)
                bwd_rm = torch.empty((p.n_in, kvp), dtype=torch.int32, device=dev)
                _lib.check(_lib.load().spc_rulebook_igemm_backward(
                    ctypes.byref(p.geom), _lib.ptr(p.indices), p.n_in, self.n_out, _lib.ptr(p.workspace),
                    p.workspace.numel(), _lib.ptr(pair_bwd), _lib.ptr(pm_bwd), _lib.ptr(ma_bwd), self.split_words,
                    self.n_split, int(bool(self.do_sort)), _lib.ptr(bwd_rm), _lib.current_stream(dev)))
                pair_bwd._spc_rowmajor = bwd_rm
            self.value = (pair_bwd, [pm_bwd[s] for s in range(self.n_split)],
                          [ma_bwd[s] for s in range(self.n_split)])
            self.p = None  # the workspace is no longer needed
        return self.value


_tls = threading.local()


@contextlib.contextmanager
def deferred_backward(defer):
    """``defer``: a DeferredBackward (build the input-side tables on its stream), the
    string "late" (do not build them; attach a LateTables to the result) or None."""
    old = getattr(_tls, "defer", None)
    _tls.defer = defer
    try:
        yield defer
    finally:
        _tls.defer = old


def igemm_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                transpose, is_train, is_mask_split, do_sort=True, num_out_act_bound=-1):
    """Reference: igemm_pairs, _impl/pairs.py:281-426.  Same 9-tuple:
    ``(out_inds, indice_num_per_loc, pair_fwd, pair_bwd, pair_mask_fwd_splits,
    pair_mask_bwd_splits, mask_argsort_fwd_splits, mask_argsort_bwd_splits, masks)``."""
    p = _prepare(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                 transpose)
    kv = p.kv
    if is_mask_split and kv > 32:
        raise AssertionError("Not Implemented")
    dev = p.indices.device
    ndim = len(spatial_shape)
    n_out = p.n_out
    if not subm and num_out_act_bound > 0 and n_out > num_out_act_bound:
        n_out = int(num_out_act_bound)
    masks = _split_masks(kv, is_mask_split)
    n_split = len(masks)
    mic = (kv + 31) // 32
    want_bwd = bool(is_train)
    want_bwd_masks = want_bwd and not subm
    with torch.cuda.device(dev):
        out_inds = indices if subm else torch.empty((n_out, ndim + 1), dtype=torch.int32, device=dev)
        pair_fwd = torch.empty((kv, n_out), dtype=torch.int32, device=dev)
        pair_bwd = torch.empty((kv, p.n_in), dtype=torch.int32, device=dev) if want_bwd else None
        pm_fwd = torch.empty((n_split, n_out, mic), dtype=torch.int32, device=dev)
        ma_fwd = torch.empty((n_split, n_out), dtype=torch.int32, device=dev)
        pm_bwd = ma_bwd = None
        if want_bwd_masks:
            pm_bwd = torch.empty((n_split, p.n_in, mic), dtype=torch.int32, device=dev)
            ma_bwd = torch.empty((n_split, p.n_in), dtype=torch.int32, device=dev)
        # row-major copies for the GEMM kernels, carried as attributes of the tables
        kvp = (kv + 3) // 4 * 4
        fwd_rm = torch.empty((n_out, kvp), dtype=torch.int32, device=dev)
        bwd_rm = torch.empty((p.n_in, kvp), dtype=torch.int32, device=dev) if want_bwd else None
        split_words = (ctypes.c_uint32 * n_split)(*[int(m[0]) for m in masks])
        defer = getattr(_tls, "defer", None) if want_bwd_masks else None
        late = None
        if defer == "late":
            # the forward half only; the other half waits until somebody reads it
            late = LateTables(p, n_out, None, n_split, do_sort, mic)
            want_bwd = want_bwd_masks = False
            pair_bwd = pm_bwd = ma_bwd = bwd_rm = None
            defer = None
        lib = _lib.load()
        _lib.check(lib.spc_rulebook_igemm(
            ctypes.byref(p.geom), _lib.ptr(p.indices), p.n_in, n_out, _lib.ptr(p.workspace),
            p.workspace.numel(), None if subm else _lib.ptr(out_inds), _lib.ptr(pair_fwd),
            None if defer else _lib.ptr(pair_bwd), _lib.ptr(pm_fwd), _lib.ptr(ma_fwd),
            None if defer else _lib.ptr(pm_bwd), None if defer else _lib.ptr(ma_bwd),
            split_words, n_split, int(bool(do_sort)), _lib.ptr(fwd_rm), None if defer else _lib.ptr(bwd_rm),
            _lib.current_stream(dev)))
        if defer is not None:
            # the input-side tables follow on the other stream, once the forward half is done
            fwd_done = torch.cuda.Event()
            fwd_done.record()
            late = [pair_bwd, pm_bwd, ma_bwd, bwd_rm]
            for t in late + [p.workspace, p.indices]:
                t.record_stream(defer.stream)
            with torch.cuda.stream(defer.stream):
                defer.stream.wait_event(fwd_done)
                _lib.check(lib.spc_rulebook_igemm_backward(
                    ctypes.byref(p.geom), _lib.ptr(p.indices), p.n_in, n_out, _lib.ptr(p.workspace),
                    p.workspace.numel(), _lib.ptr(pair_bwd), _lib.ptr(pm_bwd), _lib.ptr(ma_bwd), split_words,
                    n_split, int(bool(do_sort)), _lib.ptr(bwd_rm), _lib.current_stream(dev)))
                done = torch.cuda.Event()
                done.record()
            defer.pending.append((done, late))
        npl = torch.zeros(kv, dtype=torch.int32, device=dev)
        pair_fwd._spc_rowmajor = fwd_rm
        if late is not None:
            late.split_words = split_words
            pair_fwd._spc_late = late
        if want_bwd:
            pair_bwd._spc_rowmajor = bwd_rm
    pb = pair_bwd if want_bwd else torch.Tensor()
    pm_fwd_splits = [pm_fwd[s] for s in range(n_split)]
    ma_fwd_splits = [ma_fwd[s] for s in range(n_split)]
    if want_bwd_masks:
        pm_bwd_splits = [pm_bwd[s] for s in range(n_split)]
        ma_bwd_splits = [ma_bwd[s] for s in range(n_split)]
    else:
        pm_bwd_splits, ma_bwd_splits = [], []
    return (out_inds, npl, pair_fwd, pb, pm_fwd_splits, pm_bwd_splits, ma_fwd_splits, ma_bwd_splits, masks)


def native_pair_to_tables(pair, indice_pair_num, n_in, n_out, inverse, need_bwd=True):
    """Reference: native_pair_to_tables, _impl/pairs.py:429-469 (including the
    memoisation on the pair tensor; ``indice_pair_num`` is accepted and ignored)."""
    key = (int(n_in), int(n_out), bool(inverse))
    cache = getattr(pair, "_spconv_b200_tables", None)
    if cache is None:
        cache = {}
        pair._spconv_b200_tables = cache
    pf, pb = cache.get(key, (None, None))
    if pf is None or (need_bwd and pb is None):
        dev = pair.device
        kv, n_pair = int(pair.shape[1]), int(pair.shape[2])
        src = pair if pair.is_contiguous() else pair.contiguous()
        with torch.cuda.device(dev):
            pf = torch.empty((kv, int(n_out)), dtype=torch.int32, device=dev)
            pb = torch.empty((kv, int(n_in)), dtype=torch.int32, device=dev) if need_bwd else None
            _lib.check(_lib.load().spc_native_to_tables(
                _lib.ptr(src), kv, n_pair, int(bool(inverse)), _lib.ptr(pf), int(n_out), _lib.ptr(pb),
                int(n_in), _lib.current_stream(dev)))
        cache[key] = (pf, pb)
    return pf, pb


def rowmajor_of(pair_table):
    """Row-major copy [n, kvp] of a pair table [kv, n] for the GEMM kernels:
    the one the rulebook attached, or one built (and memoised on the tensor) now."""
    rm = getattr(pair_table, "_spc_rowmajor", None)
    if rm is None:
        kv, n = int(pair_table.shape[0]), int(pair_table.shape[1])
        dev = pair_table.device
        src = pair_table if pair_table.is_contiguous() else pair_table.contiguous()
        with torch.cuda.device(dev):
            rm = torch.empty((n, (kv + 3) // 4 * 4), dtype=torch.int32, device=dev)
            _lib.check(_lib.load().spc_pairs_to_rowmajor(_lib.ptr(src), kv, n, _lib.ptr(rm), _lib.current_stream(dev)))
        try:
            pair_table._spc_rowmajor = rm
        except AttributeError:
            pass
    return rm
