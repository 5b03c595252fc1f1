"""Rulebook parity on the GPU, through the C ABI: bit-exact against the
vectors the reference produced and against the CPU oracle on larger seeded
inputs (no canonicalisation needed: the CUDA path reproduces the reference's
row numbering)."""

import numpy as np
import pytest
import torch

from conftest import rulebook_case_names
from gpu_util import DEV, check_igemm_against, to_np, unique_coords
from oracle import rulebook as orb

pytestmark = pytest.mark.gpu


def _pairs():
    from spconv_triton_b200.pytorch._impl import pairs

    return pairs


@pytest.mark.parametrize("name", rulebook_case_names())
def test_igemm_matches_reference_vectors(ref_ops, name):
    spec = ref_ops.rulebooks[name]
    a, ig = spec["args"], spec["igemm"]
    idx = torch.from_numpy(ref_ops.rb(name, "indices")).to(DEV)
    res = _pairs().igemm_pairs(idx, a["batch_size"], a["spatial_shape"], a["ksize"], a["stride"], a["padding"],
                               a["dilation"], a["out_padding"], a["subm"], a["transpose"], ig["is_train"],
                               ig["is_mask_split"], ig["do_sort"], ig["num_out_act_bound"])
    g = lambda k: ref_ops.rb(name, k)  # noqa: E731
    n_split = 2 if ig["is_mask_split"] else 1
    has_bwd_masks = ref_ops.rb_has(name, "ig_pm_bwd0")
    exp = (g("ig_out_inds"), g("ig_npl"), g("ig_pair_fwd"), g("ig_pair_bwd"),
           [g(f"ig_pm_fwd{i}") for i in range(n_split)],
           [g(f"ig_pm_bwd{i}") for i in range(n_split)] if has_bwd_masks else [],
           [g(f"ig_ma_fwd{i}") for i in range(n_split)],
           [g(f"ig_ma_bwd{i}") for i in range(n_split)] if has_bwd_masks else [],
           [g("ig_masks")])
    check_igemm_against(res, exp, a["subm"], idx.shape[0])
    if a["subm"]:
        assert res[0] is idx  # subm returns the input indices object itself


@pytest.mark.parametrize("name", rulebook_case_names())
def test_native_matches_reference_vectors(ref_ops, name):
    if not ref_ops.rb_has(name, "nat_pair"):
        pytest.skip("no Native vectors for this variant")
    a = ref_ops.rulebooks[name]["args"]
    idx = torch.from_numpy(ref_ops.rb(name, "indices")).to(DEV)
    P = _pairs()
    out_inds, pair, npl = P.native_pairs(idx, a["batch_size"], a["spatial_shape"], a["ksize"], a["stride"],
                                         a["padding"], a["dilation"], a["out_padding"], a["subm"],
                                         a["transpose"])
    np.testing.assert_array_equal(to_np(out_inds), ref_ops.rb(name, "nat_out_inds"))
    np.testing.assert_array_equal(to_np(pair), ref_ops.rb(name, "nat_pair"))
    np.testing.assert_array_equal(to_np(npl), ref_ops.rb(name, "nat_npl"))
    for inverse in (False, True):
        n_in, n_out = idx.shape[0], out_inds.shape[0]
        if inverse:
            n_in, n_out = n_out, n_in
        pf, pb = P.native_pair_to_tables(pair.clone(), npl, n_in, n_out, inverse)
        np.testing.assert_array_equal(to_np(pf), ref_ops.rb(name, f"nat_tables_fwd_inv{int(inverse)}"))
        np.testing.assert_array_equal(to_np(pb), ref_ops.rb(name, f"nat_tables_bwd_inv{int(inverse)}"))


BIG = [
    # shape, batch, n, ksize, stride, pad, dil, opad, subm, transpose
    ([41, 400, 352], 4, 60000, [3, 3, 3], [1, 1, 1], [1, 1, 1], [1, 1, 1], [0, 0, 0], True, False),
    ([41, 400, 352], 4, 60000, [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [0, 0, 0], False, False),
    ([64, 64, 64], 2, 50000, [2, 2, 2], [2, 2, 2], [0, 0, 0], [1, 1, 1], [0, 0, 0], False, False),
    ([40, 40, 40], 2, 20000, [3, 3, 3], [1, 1, 1], [0, 0, 0], [1, 1, 1], [0, 0, 0], False, False),
    ([20, 24, 28], 2, 6000, [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [1, 1, 1], False, True),
    ([48, 48, 48], 2, 30000, [5, 5, 5], [1, 1, 1], [2, 2, 2], [1, 1, 1], [0, 0, 0], True, False),
    ([20, 20, 20, 20], 2, 20000, [3, 3, 3, 3], [1, 1, 1, 1], [1, 1, 1, 1], [1, 1, 1, 1], [0, 0, 0, 0], True, False),
    ([512, 600], 3, 40000, [3, 3], [2, 2], [1, 1], [1, 1], [0, 0], False, False),
    ([5000], 4, 3000, [5], [3], [2], [1], [0], False, False),
    # grids between 2^27.6 and 2^31 cells: too large for an input bitmap, 32-bit keys, hash table only
    ([1000, 1000, 500], 2, 50000, [3, 3, 3], [1, 1, 1], [1, 1, 1], [1, 1, 1], [0, 0, 0], True, False),
    ([1000, 1000, 500], 2, 50000, [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [0, 0, 0], False, False),
]


@pytest.mark.parametrize("order", ["given", "ascending"])
@pytest.mark.parametrize("case", range(len(BIG)))
def test_igemm_and_native_match_oracle_on_larger_inputs(case, order):
    """``ascending``: rows sorted by linear coordinate, as the outputs of an earlier layer are; the
    library then numbers input rows through its bitmap instead of the hash table."""
    shape, batch, n, k, s, p, d, op, subm, tr = BIG[case]
    if int(np.prod(shape)) > 1 << 27:
        # a dense cluster in the far corner of a huge grid: large keys, and neighbours that exist
        idx_np = unique_coords(500 + case, n, batch, [40, 40, 40])
        idx_np[:, 1:] += np.array(shape, np.int32) - 40
    else:
        idx_np = unique_coords(500 + case, n, batch, shape)
    if order == "ascending":
        lin = np.zeros(idx_np.shape[0], np.int64)
        for col, extent in enumerate([batch, *shape]):
            lin = lin * extent + idx_np[:, col]
        idx_np = np.ascontiguousarray(idx_np[np.argsort(lin)])
    idx = torch.from_numpy(idx_np).to(DEV)
    P = _pairs()
    kv = int(np.prod(k))
    algo_split = False
    res = P.igemm_pairs(idx, batch, shape, k, s, p, d, op, subm, tr, True, algo_split)
    exp = orb.igemm_pairs(idx_np, batch, shape, k, s, p, d, op, subm, tr, True, algo_split)
    check_igemm_against(res, exp, subm, n)
    if kv <= 27 or n <= 20000:
        out_inds, pair, npl = P.native_pairs(idx, batch, shape, k, s, p, d, op, subm, tr)
        e_out, e_pair, e_npl = orb.native_pairs(idx_np, batch, shape, k, s, p, d, op, subm, tr)
        np.testing.assert_array_equal(to_np(out_inds), e_out)
        np.testing.assert_array_equal(to_np(pair), e_pair)
        np.testing.assert_array_equal(to_np(npl), e_npl)


def test_int64_linearisation_translation_invariance():
    """batch * volume >= 2^31 switches the hash tables to 64-bit keys; the
    rulebook of a point set must not change when the set is translated far
    into such a grid (the property the reference tests in
    tests/test_int64_linearize.py)."""
    shape_small, shape_big = [64, 64, 32], [2048, 2048, 512]
    idx_np = unique_coords(77, 5000, 2, shape_small)
    far = idx_np.copy()
    far[:, 1:] += np.array([1980, 1976, 472], dtype=np.int32)  # even shift keeps stride-2 parity
    P = _pairs()
    for subm, s, p in ((True, [1, 1, 1], [1, 1, 1]), (False, [2, 2, 2], [1, 1, 1])):
        a = P.igemm_pairs(torch.from_numpy(idx_np).to(DEV), 2, shape_small, [3, 3, 3], s, p, [1, 1, 1],
                          [0, 0, 0], subm, False, True, False)
        b = P.igemm_pairs(torch.from_numpy(far).to(DEV), 2, shape_big, [3, 3, 3], s, p, [1, 1, 1], [0, 0, 0],
                          subm, False, True, False)
        exp = orb.igemm_pairs(far, 2, shape_big, [3, 3, 3], s, p, [1, 1, 1], [0, 0, 0], subm, False, True, False)
        check_igemm_against(b, exp, subm, 5000)
        if subm:  # neighbours are unchanged by the shift, so the tables are identical
            np.testing.assert_array_equal(to_np(a[2]), to_np(b[2]))


def test_deterministic_and_reusable_workspace():
    idx = torch.from_numpy(unique_coords(5, 30000, 2, [41, 200, 176])).to(DEV)
    P = _pairs()
    args = (idx, 2, [41, 200, 176], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [0, 0, 0], False, False, True, False)
    r1 = P.igemm_pairs(*args)
    r2 = P.igemm_pairs(*args)
    for a, b in zip(r1[:4], r2[:4]):
        assert torch.equal(a, b)
    assert torch.equal(r1[4][0], r2[4][0]) and torch.equal(r1[6][0], r2[6][0])


def test_host_side_errors():
    P = _pairs()
    idx = torch.from_numpy(unique_coords(1, 50, 1, [8, 8, 8])).to(DEV)
    three = lambda v: [v] * 3  # noqa: E731
    with pytest.raises(ValueError, match="N > 0"):
        P.igemm_pairs(idx[:0], 1, [8, 8, 8], three(3), three(1), three(1), three(1), three(0), True, False, True, False)
    with pytest.raises(NotImplementedError):
        P.igemm_pairs(idx, 1, [8, 8, 8], three(2), three(1), three(0), three(1), three(0), True, False, True, False)
    with pytest.raises(ValueError, match="reach zero"):
        P.igemm_pairs(idx, 1, [8, 8, 8], three(9), three(1), three(0), three(1), three(0), False, False, True, False)
    with pytest.raises(AssertionError, match="Not Implemented"):
        P.igemm_pairs(idx, 1, [8, 8, 8], three(5), three(1), three(2), three(1), three(0), True, False, True, True)
    # every point falls outside the only window a stride-8 k=1 layer keeps
    far = idx.clone()
    far[:, 1:] = far[:, 1:] % 7 + 1
    with pytest.raises(ValueError, match="points vanished"):
        P.igemm_pairs(far, 1, [8, 8, 8], three(1), three(8), three(0), three(1), three(0), False, False, True, False)


def test_rows_outside_the_grid_are_skipped_and_reported():
    """A batch index >= batch_size or a coordinate outside spatial_shape must not become a bitmap or
    table index.  Strided layers read their counters on the host and raise at once; submanifold
    layers have no host read: the row gets no pairs and the device status word carries the error
    to the next status check."""
    from spconv_triton_b200 import _lib
    from spconv_triton_b200.pytorch._impl import gemm as G

    P = _pairs()
    shape, batch = [16, 20, 24], 2
    good = unique_coords(3, 4000, batch, shape)
    three = lambda v: [v] * 3  # noqa: E731
    G.check_device_status()
    for bad in ([2, 1, 1, 1], [0, 16, 0, 0], [0, -1, 3, 3], [-1, 0, 0, 0], [1, 5, 5, 1 << 20]):
        rows = good.copy()
        rows[123] = bad
        idx = torch.from_numpy(rows).to(DEV)
        with pytest.raises(_lib.SpconvB200Error, match="outside batch_size") as e:
            P.igemm_pairs(idx, batch, shape, three(3), three(2), three(1), three(1), three(0), False, False, True, False)
        assert e.value.status == _lib.SPC_ERR_INVALID_ARGUMENT
        res = P.igemm_pairs(idx, batch, shape, three(3), three(1), three(1), three(1), three(0), True, False, True, False)
        assert bool((res[2][:, 123] == -1).all()) and bool((res[3][:, 123] == -1).all())
        assert not bool((res[2] == 123).any())
        with pytest.raises(_lib.SpconvB200Error, match="outside batch_size"):
            G.check_device_status()
        G.check_device_status()  # reported once, then clear
    # the rest of the rows are unaffected
    exp = orb.igemm_pairs(np.delete(good, 123, 0), batch, shape, three(3), three(1), three(1), three(1), three(0), True,
                          False, True, False)
    got = P.igemm_pairs(torch.from_numpy(np.delete(good, 123, 0)).to(DEV), batch, shape, three(3), three(1), three(1),
                        three(1), three(0), True, False, True, False)
    check_igemm_against(got, exp, True, good.shape[0] - 1)
