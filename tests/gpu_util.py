"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

DEV = "cuda"


def unique_coords(seed, n, batch, shape):
    """n unique (batch, *coords) int32 rows in shuffled order."""
    rng = np.random.default_rng(seed)
    vol = int(np.prod(shape))
    per = [n // batch + (1 if b < n % batch else 0) for b in range(batch)]
    rows = []
    for b, m in enumerate(per):
        lin = rng.choice(vol, size=m, replace=False)
        c = np.stack(np.unravel_index(lin, shape), axis=1)
        rows.append(np.concatenate([np.full((m, 1), b), c], axis=1))
    out = np.concatenate(rows, 0).astype(np.int32)
    return out[rng.permutation(out.shape[0])]


def to_np(t):
    return t.detach().cpu().numpy()


def rel_err(actual, expected):
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, (a.shape, e.shape)
    if e.size == 0:
        return 0.0
    return float(np.abs(a - e).max()) / max(float(np.abs(e).max()), 1e-30)


def check_igemm_against(res, exp, subm, n_in):
    """res: 9-tuple of torch tensors from the C-ABI path; exp: 9-tuple of numpy
    arrays from the oracle / the reference.  Bit-exact on every member."""
    out_inds, npl, pf, pb, pmf, pmb, maf, mab, masks = res
    e_out, e_npl, e_pf, e_pb, e_pmf, e_pmb, e_maf, e_mab, e_masks = exp
    np.testing.assert_array_equal(to_np(out_inds), e_out)
    np.testing.assert_array_equal(to_np(npl), e_npl)
    np.testing.assert_array_equal(to_np(pf), e_pf)
    if e_pb is None or (hasattr(e_pb, "size") and e_pb.size == 0):
        assert pb.numel() == 0
    else:
        np.testing.assert_array_equal(to_np(pb), e_pb)
    assert len(pmf) == len(e_pmf) and len(pmb) == len(e_pmb)
    for a, e in zip(list(pmf) + list(pmb) + list(maf) + list(mab),
                    list(e_pmf) + list(e_pmb) + list(e_maf) + list(e_mab)):
        np.testing.assert_array_equal(to_np(a), e)
    np.testing.assert_array_equal(np.concatenate(masks), np.concatenate(e_masks))
