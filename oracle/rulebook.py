"""CPU oracle: rulebook (indice-pair) generation, restated in numpy.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Each function follows the reference file it cites (paths are inside the
reference project):

* output-shape formulas ........ spconv_triton/pytorch/_impl/pairs.py:59-88
* kernel-offset enumeration ..... spconv_triton/pytorch/_impl/pairs.py:43-48
* candidates / membership ....... spconv_triton/pytorch/_impl/pairs.py:126-220 and
                                  spconv_triton/pytorch/_impl/pair_kernels.py:38-94,298-446
* Native [2,kv,N] rulebook ...... spconv_triton/pytorch/_impl/pairs.py:223-278
* implicit-gemm tables + masks .. spconv_triton/pytorch/_impl/pairs.py:281-426
* Native -> tables .............. spconv_triton/pytorch/_impl/pairs.py:429-469

All linear coordinates are computed in int64; the reference switches between
int32 and int64 but states that both agree on every entry it consumes
(pairs.py:166-171), so int64 is the faithful superset.
"""

from __future__ import annotations

import numpy as np

POINT_VANISH_MSG = (
    "Your points vanished here, this usually happens when you provide "
    "conv params that may ignore some input points. Example: "
    "spatial_shape={}, ksize={}, stride={}, padding={}, dilation={}"
)


def conv_output_size(input_size, kernel_size, stride, padding, dilation):
    """pairs.py:59-70."""
    out = []
    for s, k, st, p, d in zip(input_size, kernel_size, stride, padding, dilation):
        out.append(1 if k == -1 else (s + 2 * p - d * (k - 1) - 1) // st + 1)
    return out


def deconv_output_size(input_size, kernel_size, stride, padding, dilation, output_padding):
    """pairs.py:73-88 (dilation does not enter the reference's formula)."""
    out = []
    for s, k, st, p, op in zip(input_size, kernel_size, stride, padding, output_padding):
        if k == -1:
            raise ValueError("deconv don't support kernel_size < 0")
        out.append((s - 1) * st - 2 * p + k + op)
    return out


def rows_in_grid(indices, batch_size, spatial_shape):
    """Boolean [N]: rows whose batch index lies in [0, batch_size) and whose
    coordinates lie inside ``spatial_shape``.  The reference linearises whatever
    it is given (spconv_triton/pytorch/_impl/pairs.py:91-95); the CUDA path
    rejects the rows for which this is False, because their linear coordinate
    would index outside its occupancy bitmaps."""
    idx = np.asarray(indices)
    ok = (idx[:, 0] >= 0) & (idx[:, 0] < int(batch_size))
    for d, extent in enumerate(spatial_shape):
        ok &= (idx[:, d + 1] >= 0) & (idx[:, d + 1] < int(extent))
    return ok


def kernel_offsets(ksize):
    """[kv, ndim] offsets, row-major with the last dimension fastest (pairs.py:43-48)."""
    grids = np.meshgrid(*[np.arange(k, dtype=np.int64) for k in ksize], indexing="ij")
    return np.stack([g.reshape(-1) for g in grids], axis=1)


def linearize(indices, shape):
    """Batch-major, then row-major over ``shape`` (pairs.py:91-95)."""
    idx = np.asarray(indices, dtype=np.int64)
    lin = idx[:, 0].copy()
    for i, s in enumerate(shape):
        lin = lin * int(s) + idx[:, i + 1]
    return lin


def delinearize(lin, shape):
    """Inverse of :func:`linearize`; returns int32 [n, ndim+1] (pairs.py:98-111)."""
    lin = np.asarray(lin, dtype=np.int64)
    ndim = len(shape)
    out = np.empty((lin.shape[0], ndim + 1), dtype=np.int32)
    rem = lin
    for i in range(ndim - 1, -1, -1):
        out[:, i + 1] = rem % shape[i]
        rem = rem // shape[i]
    out[:, 0] = rem
    return out


class Candidates:
    def __init__(self, valid, out_row, out_inds, out_shape, n_out, kv):
        self.valid = valid
        self.out_row = out_row
        self.out_inds = out_inds
        self.out_shape = out_shape
        self.n_out = n_out
        self.kv = kv


def compute_candidates(indices, batch_size, spatial_shape, ksize, stride, padding,
                       dilation, out_padding, subm, transpose):
    """valid[kv,N], out_row[kv,N] (meaningful where valid), output indices.

    pairs.py:126-220; the per-dimension arithmetic is pair_kernels.py:66-91.
    """
    indices = np.asarray(indices)
    ndim = len(spatial_shape)
    n = indices.shape[0]
    kv = int(np.prod(ksize))
    if n == 0:
        raise ValueError("N > 0 assert: sparse tensor has no points")
    if any(k <= 0 for k in ksize):
        raise ValueError(f"kernel size {list(ksize)} not supported by pair gen")
    if subm:
        if any(k % 2 == 0 for k in ksize):
            raise NotImplementedError("subm convolution requires odd kernel sizes")
        out_shape = list(spatial_shape)
    elif transpose:
        out_shape = deconv_output_size(spatial_shape, ksize, stride, padding, dilation, out_padding)
    else:
        out_shape = conv_output_size(spatial_shape, ksize, stride, padding, dilation)
    if any(x <= 0 for x in out_shape):
        raise ValueError(
            f"your out spatial shape {out_shape} reach zero!!! input shape: {list(spatial_shape)}"
        )
    if subm:
        pad = [(ksize[i] // 2) * dilation[i] for i in range(ndim)]
        st = [1] * ndim
    else:
        pad = list(padding)
        st = list(stride)

    idx = indices.astype(np.int64)
    offs = kernel_offsets(ksize)  # [kv, ndim]
    acc = np.broadcast_to(idx[None, :, 0], (kv, n)).copy()
    valid = np.ones((kv, n), dtype=bool)
    for d in range(ndim):
        c = idx[None, :, d + 1]
        off = offs[:, d][:, None] * int(dilation[d])
        if transpose:
            o = c * int(st[d]) + off - int(pad[d])
            valid &= (o >= 0) & (o < out_shape[d])
            contrib = o
        else:
            num = c + int(pad[d]) - off
            q = np.floor_divide(num, int(st[d]))
            valid &= (num >= 0) & (num - q * int(st[d]) == 0) & (q < out_shape[d])
            contrib = q
        acc = acc * int(out_shape[d]) + contrib
    out_lin = acc

    if subm:
        in_lin = linearize(idx, spatial_shape)
        sort_idx = np.argsort(in_lin, kind="stable")
        sorted_lin = in_lin[sort_idx]
        pos = np.searchsorted(sorted_lin, out_lin.reshape(-1), side="left")
        pos_c = np.minimum(pos, n - 1)
        found = (pos < n) & (sorted_lin[pos_c] == out_lin.reshape(-1))
        out_row = sort_idx[pos_c].reshape(kv, n).astype(np.int32)
        valid = valid & found.reshape(kv, n)
        return Candidates(valid, out_row, indices, out_shape, n, kv)

    uniq = np.unique(out_lin[valid])
    n_out = int(uniq.shape[0])
    if n_out == 0:
        raise ValueError(POINT_VANISH_MSG.format(list(spatial_shape), list(ksize), list(stride),
                                                 list(padding), list(dilation)))
    out_row = np.searchsorted(uniq, out_lin.reshape(-1), side="left").reshape(kv, n)
    out_row = np.where(valid, out_row, 0).astype(np.int32)
    out_inds = delinearize(uniq, out_shape)
    return Candidates(valid, out_row, out_inds, out_shape, n_out, kv)


def native_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation,
                 out_padding, subm, transpose):
    """Native rulebook: (out_inds, pair[2,kv,N] int32 (-1 fill), indice_num_per_loc[kv]).

    pairs.py:223-278: per offset the valid input rows in ascending order, with
    their output rows; subm zeroes the counts of offsets >= kv//2 but keeps
    the pair content.
    """
    cand = compute_candidates(indices, batch_size, spatial_shape, ksize, stride, padding,
                              dilation, out_padding, subm, transpose)
    kv, n = cand.valid.shape
    pair = np.full((2, kv, n), -1, dtype=np.int32)
    counts = cand.valid.sum(1).astype(np.int32)
    for k in range(kv):
        j = np.nonzero(cand.valid[k])[0]
        pair[0, k, : j.shape[0]] = j
        pair[1, k, : j.shape[0]] = cand.out_row[k, j]
    if subm:
        npl = np.where(np.arange(kv) < kv // 2, counts, 0).astype(np.int32)
    else:
        npl = counts
    return cand.out_inds, pair, npl


def split_masks(kv, is_mask_split):
    """pairs.py:344-352."""
    if is_mask_split:
        half = kv // 2
        remain = kv - half
        one = np.array([1], dtype=np.uint64)
        first = (one << np.uint64(remain)) - np.uint64(1)
        second = ((one << np.uint64(half)) - np.uint64(1)) << np.uint64(remain)
        return [first.astype(np.uint32), second.astype(np.uint32)]
    return [np.array([0xFFFFFFFF], dtype=np.uint32)]


def mask_words(pair_table, kv):
    """[n, ceil(kv/32)] int64; bit k%32 of word k//32 set iff pair_table[k,row] >= 0.

    pair_kernels.py:159-183.
    """
    n = pair_table.shape[1]
    mic = (kv + 31) // 32
    words = np.zeros((n, mic), dtype=np.int64)
    for k in range(kv):
        words[:, k // 32] |= (pair_table[k] >= 0).astype(np.int64) << (k % 32)
    return words


def sorted_masks(pair_table, kv, masks, do_sort):
    """Per split: (pair_mask [n, mic] int32 sorted ascending as unsigned, stable;
    multi-word = lexicographic with the highest word most significant;
    mask_argsort [n] int32 = original row of each sorted slot).  pairs.py:356-392.
    """
    n = pair_table.shape[1]
    mic = (kv + 31) // 32
    words = mask_words(pair_table, kv)
    pm_splits, arg_splits = [], []
    for m in masks:
        mval = int(np.asarray(m).astype(np.int64)[0])
        mw = words.copy()
        mw[:, 0] &= mval
        if do_sort:
            # np.lexsort: last key is the primary one, and the sort is stable.
            args = np.lexsort(tuple(mw[:, w] for w in range(mic))) if n > 0 else np.zeros(0, np.int64)
            vals = mw[args]
        else:
            args = np.arange(n)
            vals = mw
        pm = (vals & 0xFFFFFFFF).astype(np.uint32).view(np.int32).reshape(n, mic)
        pm_splits.append(pm)
        arg_splits.append(args.astype(np.int32))
    return pm_splits, arg_splits


def igemm_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation,
                out_padding, subm, transpose, is_train, is_mask_split, do_sort=True,
                num_out_act_bound=-1):
    """Implicit-gemm rulebook, same 9-tuple as pairs.py:281-426 (numpy arrays;
    an absent pair_bwd is returned as ``None``)."""
    indices = np.asarray(indices)
    n = indices.shape[0]
    cand = compute_candidates(indices, batch_size, spatial_shape, ksize, stride, padding,
                              dilation, out_padding, subm, transpose)
    kv = cand.kv
    if is_mask_split and kv > 32:
        raise AssertionError("Not Implemented")
    n_out = cand.n_out
    valid = cand.valid
    out_inds = cand.out_inds
    if not subm and num_out_act_bound > 0 and n_out > num_out_act_bound:
        n_out = num_out_act_bound
        out_inds = out_inds[:n_out]
        valid = valid & (cand.out_row < n_out)

    pair_fwd = np.full((kv, n_out), -1, dtype=np.int32)
    kk, jj = np.nonzero(valid)
    pair_fwd[kk, cand.out_row[kk, jj]] = jj.astype(np.int32)
    pair_bwd = None
    if is_train:
        pair_bwd = np.where(valid, cand.out_row, -1).astype(np.int32)

    npl = np.zeros(kv, dtype=np.int32)
    masks = split_masks(kv, is_mask_split)
    pm_fwd, ma_fwd = sorted_masks(pair_fwd, kv, masks, do_sort)
    if is_train and not subm:
        pm_bwd, ma_bwd = sorted_masks(pair_bwd, kv, masks, do_sort)
    else:
        pm_bwd, ma_bwd = [], []
    if subm:
        out_inds = indices
    return out_inds, npl, pair_fwd, pair_bwd, pm_fwd, pm_bwd, ma_fwd, ma_bwd, masks


def native_pair_to_tables(pair, n_in, n_out, inverse, need_bwd=True):
    """pairs.py:429-469: content-based (>= 0) validity; ``inverse`` swaps roles."""
    pair = np.asarray(pair)
    pair_in = pair[int(bool(inverse))]
    pair_out = pair[int(not inverse)]
    kv = pair_in.shape[0]
    valid = (pair_in >= 0) & (pair_out >= 0)
    kk, pp = np.nonzero(valid)
    pf = np.full((kv, n_out), -1, dtype=np.int32)
    pf[kk, pair_out[kk, pp]] = pair_in[kk, pp]
    pb = None
    if need_bwd:
        pb = np.full((kv, n_in), -1, dtype=np.int32)
        pb[kk, pair_in[kk, pp]] = pair_out[kk, pp]
    return pf, pb
