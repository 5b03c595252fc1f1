"""The numpy restatement of the point-to-voxel step against the reference's own
vectors: the frozen CPU cases of tests/data/golden_ext_p2v.pt (bitwise, as the
reference's tests/test_ext_p2v.py:13-29 checks them) and cases produced by the
reference class itself (tests/golden/make_golden_p2v.py)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle.voxelize import point_to_voxel

GOLD = torch.load(Path(__file__).parent / "golden" / "ref_p2v.pt", map_location="cpu", weights_only=False)
FROZEN_CPU = [c for c in GOLD["frozen"] if c["kind"] == "p2v_cpu"]
FROZEN_CANON = [c for c in GOLD["frozen"] if c["kind"] == "p2v_gpu_canon"]


def canon(idx, vox, npv):
    """Voxels ordered by coordinate, the points of a voxel ordered by a key over
    their features (the canonical form of the reference's tests/helpers.py:442-465)."""
    idx = np.asarray(idx).astype(np.int64)
    vox = np.asarray(vox).astype(np.float64)
    npv = np.asarray(npv).astype(np.int64)
    order = np.lexsort(idx.T[::-1])
    idx, vox, npv = idx[order], vox[order].copy(), npv[order]
    for i in range(vox.shape[0]):
        n = int(min(npv[i], vox.shape[1]))
        pts = vox[i, :n].copy()
        key = pts[:, 0].copy()
        for d in range(1, pts.shape[1]):
            key = key * 131071.0 + pts[:, d]
        vox[i, :n] = pts[np.argsort(key, kind="stable")]
    return idx, vox, npv


def check(out, expect, mean_tol=0.0):
    vox, idx, npv, pcvid = out
    np.testing.assert_array_equal(idx, expect["indices"].numpy())
    np.testing.assert_array_equal(npv, expect["num_per_voxel"].numpy())
    np.testing.assert_array_equal(pcvid, expect["pc_voxel_id"].numpy())
    if mean_tol:
        np.testing.assert_allclose(vox, expect["voxels"].numpy(), rtol=0, atol=mean_tol)
    else:
        np.testing.assert_array_equal(vox, expect["voxels"].numpy())


@pytest.mark.parametrize("case", FROZEN_CPU, ids=lambda c: c["id"])
def test_frozen_cpu_cases_bitwise(case):
    check(point_to_voxel(case["points"].numpy(), **case["ctor"]), case["expect"])


@pytest.mark.parametrize("case", FROZEN_CANON, ids=lambda c: c["id"])
def test_frozen_canonical_cases(case):
    vox, idx, npv, _ = point_to_voxel(case["points"].numpy(), **case["ctor"])
    i, v, n = canon(idx, vox, npv)
    e = case["expect"]
    np.testing.assert_array_equal(i, e["indices_canon"].numpy())
    np.testing.assert_array_equal(n, e["num_per_voxel_canon"].numpy())
    if e["check_contents"]:
        np.testing.assert_allclose(v, e["voxels_canon"].numpy(), rtol=0, atol=1e-5)


@pytest.mark.parametrize("case", GOLD["generated"], ids=lambda c: c["id"])
def test_generated_cases(case):
    # the oracle is stateless: only calls that start from cleared buffers compare
    for (clear, mean), expect in zip(case["calls"], case["expect"]):
        if not clear:
            continue
        out = point_to_voxel(case["points"].numpy(), empty_mean=mean, **case["ctor"])
        check(out, expect, mean_tol=1e-6 if mean else 0.0)
