"""Sparse pooling parity on the GPU through the C ABI."""

import numpy as np
import pytest
import torch

from conftest import feature_case_names
from gpu_util import DEV, rel_err, to_np, unique_coords
from oracle import features as of
from oracle import rulebook as orb

pytestmark = pytest.mark.gpu
POOL_CASES = [n for n in feature_case_names() if n.startswith(("max", "avg"))]
TOL = {"float32": 1e-6, "float16": 1e-3, "float64": 1e-12, "bfloat16": 8e-3}


def _pool():
    from spconv_triton_b200.pytorch._impl import pool

    return pool


@pytest.mark.parametrize("name", POOL_CASES)
def test_matches_reference_vectors(ref_ops, name):
    spec = ref_ops.features[name]
    rb, dt = spec["rulebook"], spec["dtype"]
    g = lambda k: torch.from_numpy(ref_ops.get(f"pl/{name}/{k}"))  # noqa: E731
    pf = torch.from_numpy(ref_ops.rb(rb, "ig_pair_fwd")).to(DEV)
    pb = torch.from_numpy(ref_ops.rb(rb, "ig_pair_bwd")).to(DEV)
    feats, gout = g("features").to(DEV), g("grad_out").to(DEV)
    P = _pool()
    if name.startswith("max"):
        out = P.maxpool_forward(feats, pf, pf.shape[1])
        np.testing.assert_array_equal(to_np(out), g("out").numpy())  # comparisons only: bit-exact
        din = P.maxpool_backward(feats, out, gout, pb)
    else:
        out, cnt = P.avgpool_forward(feats, pf, pf.shape[1])
        np.testing.assert_array_equal(to_np(cnt), g("count").numpy())
        assert rel_err(to_np(out.double()), g("out").double().numpy()) <= TOL[dt]
        din = P.avgpool_backward(gout, pb, cnt)
    assert rel_err(to_np(din.double()), g("din").double().numpy()) <= TOL[dt]


# Channel counts chosen to reach every launch shape: rows of 4, 8, 16 and 32
# threads with 1, 2 or 4 vectors each (the warp-group kernel), and rows that are
# too narrow, not a power of two, or unaligned (the shared-memory kernel).
# ksize 4 stride 1 has 64 offsets: more than one 32-entry round of the table.
@pytest.mark.parametrize("dtype,channels,ksize,stride", [
    (torch.float16, 64, 2, 2), (torch.float32, 32, 2, 2), (torch.float16, 20, 2, 2), (torch.bfloat16, 16, 2, 2),
    (torch.float64, 6, 2, 2), (torch.float32, 7, 2, 2), (torch.float16, 256, 3, 1), (torch.float16, 512, 2, 2),
    (torch.bfloat16, 1024, 2, 2), (torch.float16, 32, 3, 1), (torch.float32, 48, 3, 2), (torch.float16, 96, 4, 1),
    (torch.float32, 20, 4, 1), (torch.float64, 8, 3, 1), (torch.float16, 4096, 2, 2)])
def test_matches_oracle(dtype, channels, ksize, stride):
    shape, batch, n = [32, 48, 40], 3, (40000 if channels <= 256 else 6000)
    idx_np = unique_coords(31, n, batch, shape)
    res = orb.igemm_pairs(idx_np, batch, shape, [ksize] * 3, [stride] * 3, [0] * 3, [1] * 3, [0] * 3, False, False, True, False)
    pf, pb = res[2], res[3]
    n_out = pf.shape[1]
    gen = torch.Generator().manual_seed(5)
    feats = (torch.randint(-8, 8, (n, channels), generator=gen).float() * 0.125).to(dtype)
    gout = torch.randn(n_out, channels, generator=gen).to(dtype)
    P = _pool()
    pfd, pbd = torch.from_numpy(pf).to(DEV), torch.from_numpy(pb).to(DEV)
    tol = TOL[str(dtype).split(".")[1]]
    out = P.maxpool_forward(feats.to(DEV), pfd, n_out)
    e_out = of.maxpool_forward(feats, pf, n_out)
    assert torch.equal(out.cpu(), e_out)
    din = P.maxpool_backward(feats.to(DEV), out, gout.to(DEV), pbd)
    assert rel_err(to_np(din.double()), of.maxpool_backward(feats, e_out, gout, pb).double().numpy()) <= tol
    out, cnt = P.avgpool_forward(feats.to(DEV), pfd, n_out)
    e_out, e_cnt = of.avgpool_forward(feats, pf, n_out)
    assert torch.equal(cnt.cpu(), e_cnt)
    assert rel_err(to_np(out.double()), e_out.double().numpy()) <= tol
    din = P.avgpool_backward(gout.to(DEV), pbd, cnt)
    assert rel_err(to_np(din.double()), of.avgpool_backward(gout, pb, e_cnt).double().numpy()) <= tol


def test_max_pool_is_clamped_at_zero():
    """All-negative windows give 0 because the accumulator starts at 0, the
    behaviour the reference pins in tests/test_pool.py:43-56."""
    import spconv_triton_b200.pytorch as sp

    idx = torch.tensor([[0, 0, 0, 0], [0, 0, 0, 1], [0, 2, 2, 2]], dtype=torch.int32, device=DEV)
    feats = torch.tensor([[-1.0, 2.0], [-3.0, -4.0], [-5.0, -6.0]], device=DEV)
    x = sp.SparseConvTensor(feats, idx, [4, 4, 4], 1)
    out = sp.SparseMaxPool3d(2, 2)(x)
    order = torch.argsort(out.indices[:, 1] * 100 + out.indices[:, 2] * 10 + out.indices[:, 3])
    assert out.features[order].tolist() == [[0.0, 2.0], [0.0, 0.0]]
