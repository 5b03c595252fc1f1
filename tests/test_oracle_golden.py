"""Pins the CPU oracle to the reference: every oracle function is compared with
the vectors the reference itself produced (tests/golden/ref_ops.npz).

Rulebooks must be bit-exact.  Feature results are compared within the
tolerances the hot path is specified to: 1e-5 relative (fp32), 2e-3 (fp16),
measured against the largest reference magnitude as the reference's own
calibrated goldens do.
"""

import numpy as np
import pytest
import torch

from conftest import feature_case_names, rulebook_case_names
from oracle import features as of
from oracle import rulebook as orb

TOL = {"float32": 1e-5, "float16": 2e-3, "float64": 1e-12}


def _close(actual, expected, rel, what):
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, what
    scale = max(float(np.abs(e).max()), 1e-30) if e.size else 1.0
    err = float(np.abs(a - e).max()) if e.size else 0.0
    assert err <= rel * scale, f"{what}: err {err:.3e} > {rel:.0e} * {scale:.3e}"


@pytest.mark.parametrize("name", rulebook_case_names())
def test_igemm_rulebook_bit_exact(ref_ops, name):
    spec = ref_ops.rulebooks[name]
    a, ig = spec["args"], spec["igemm"]
    idx = ref_ops.rb(name, "indices")
    res = orb.igemm_pairs(idx, a["batch_size"], a["spatial_shape"], a["ksize"], a["stride"],
                          a["padding"], a["dilation"], a["out_padding"], a["subm"], a["transpose"],
                          ig["is_train"], ig["is_mask_split"], ig["do_sort"], ig["num_out_act_bound"])
    out_inds, npl, pf, pb, pmf, pmb, maf, mab, masks = res
    np.testing.assert_array_equal(out_inds, ref_ops.rb(name, "ig_out_inds"))
    np.testing.assert_array_equal(npl, ref_ops.rb(name, "ig_npl"))
    np.testing.assert_array_equal(pf, ref_ops.rb(name, "ig_pair_fwd"))
    exp_pb = ref_ops.rb(name, "ig_pair_bwd")
    if exp_pb.size:
        np.testing.assert_array_equal(pb, exp_pb)
    else:
        assert pb is None
    for split, (m, s) in enumerate(zip(pmf, maf)):
        np.testing.assert_array_equal(m, ref_ops.rb(name, f"ig_pm_fwd{split}"))
        np.testing.assert_array_equal(s, ref_ops.rb(name, f"ig_ma_fwd{split}"))
    assert len(pmb) == sum(ref_ops.rb_has(name, f"ig_pm_bwd{i}") for i in range(2))
    for split, (m, s) in enumerate(zip(pmb, mab)):
        np.testing.assert_array_equal(m, ref_ops.rb(name, f"ig_pm_bwd{split}"))
        np.testing.assert_array_equal(s, ref_ops.rb(name, f"ig_ma_bwd{split}"))
    np.testing.assert_array_equal(np.concatenate(masks), ref_ops.rb(name, "ig_masks"))


@pytest.mark.parametrize("name", rulebook_case_names())
def test_native_rulebook_bit_exact(ref_ops, name):
    if not ref_ops.rb_has(name, "nat_pair"):
        pytest.skip("reference Native vectors not generated for this variant")
    a = ref_ops.rulebooks[name]["args"]
    idx = ref_ops.rb(name, "indices")
    out_inds, pair, npl = orb.native_pairs(idx, a["batch_size"], a["spatial_shape"], a["ksize"],
                                           a["stride"], a["padding"], a["dilation"],
                                           a["out_padding"], a["subm"], a["transpose"])
    np.testing.assert_array_equal(out_inds, ref_ops.rb(name, "nat_out_inds"))
    np.testing.assert_array_equal(pair, ref_ops.rb(name, "nat_pair"))
    np.testing.assert_array_equal(npl, ref_ops.rb(name, "nat_npl"))
    for inverse in (False, True):
        n_in, n_out = idx.shape[0], out_inds.shape[0]
        if inverse:
            n_in, n_out = n_out, n_in
        pf, pb = orb.native_pair_to_tables(pair, n_in, n_out, inverse)
        np.testing.assert_array_equal(pf, ref_ops.rb(name, f"nat_tables_fwd_inv{int(inverse)}"))
        np.testing.assert_array_equal(pb, ref_ops.rb(name, f"nat_tables_bwd_inv{int(inverse)}"))


@pytest.mark.parametrize("name", [n for n in feature_case_names() if not n.startswith(("max", "avg"))])
def test_gemm_matches_reference(ref_ops, name):
    spec = ref_ops.features[name]
    rb, dt = spec["rulebook"], spec["dtype"]
    g = lambda k: torch.from_numpy(ref_ops.get(f"ft/{name}/{k}"))  # noqa: E731
    pf = ref_ops.rb(rb, "ig_pair_fwd")
    pb = ref_ops.rb(rb, "ig_pair_bwd")
    feats, w, gout = g("features"), g("weight"), g("grad_out")
    bias = g("bias") if ref_ops.has(f"ft/{name}/bias") else None
    out = of.conv_forward(feats, w, pf, pf.shape[1], bias=bias)
    din = of.conv_backward_input(gout, w, pb, feats.shape[0])
    dw = of.conv_backward_weight(feats, gout, pf, tuple(w.shape))
    _close(out.numpy(), g("out").numpy(), TOL[dt], "out")
    _close(din.numpy(), g("din").numpy(), TOL[dt], "din")
    _close(dw.numpy(), g("dw").numpy(), TOL[dt], "dw")


@pytest.mark.parametrize("name", [n for n in feature_case_names() if n.startswith(("max", "avg"))])
def test_pool_matches_reference(ref_ops, name):
    spec = ref_ops.features[name]
    rb, dt = spec["rulebook"], spec["dtype"]
    g = lambda k: torch.from_numpy(ref_ops.get(f"pl/{name}/{k}"))  # noqa: E731
    pf = ref_ops.rb(rb, "ig_pair_fwd")
    pb = ref_ops.rb(rb, "ig_pair_bwd")
    feats, gout = g("features"), g("grad_out")
    if name.startswith("max"):
        out = of.maxpool_forward(feats, pf, pf.shape[1])
        din = of.maxpool_backward(feats, out, gout, pb)
        # comparisons only: bit-exact
        np.testing.assert_array_equal(out.numpy(), g("out").numpy())
    else:
        out, cnt = of.avgpool_forward(feats, pf, pf.shape[1])
        np.testing.assert_array_equal(cnt.numpy(), g("count").numpy())
        din = of.avgpool_backward(gout, pb, cnt)
        _close(out.numpy(), g("out").numpy(), TOL[dt], "out")
    _close(din.numpy(), g("din").numpy(), TOL[dt], "din")


def test_output_size_known_answers():
    # literals of the kind the reference pins in tests/test_ops.py:22-38
    assert orb.conv_output_size([41, 1600, 1408], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1]) == [21, 800, 704]
    assert orb.conv_output_size([10], [-1], [1], [0], [1]) == [1]
    assert orb.conv_output_size([7, 9], [3, 2], [2, 1], [1, 0], [1, 1]) == [4, 8]
    assert orb.deconv_output_size([8, 8, 8], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [1, 1, 1]) == [16, 16, 16]
    with pytest.raises(ValueError):
        orb.deconv_output_size([8], [-1], [1], [0], [1], [0])


def test_rows_in_grid():
    from oracle import rulebook as orb

    idx = np.array([[0, 0, 0, 0], [1, 15, 19, 23], [2, 1, 1, 1], [0, 16, 0, 0], [0, -1, 3, 3], [-1, 0, 0, 0]], np.int32)
    assert orb.rows_in_grid(idx, 2, [16, 20, 24]).tolist() == [True, True, False, False, False, False]
