"""Parity at the benchmark configurations' full sizes, through properties that
do not need the (slow) CPU oracle:

* rulebook: output coordinates strictly ascending in linear order (= sorted and
  unique), pair_fwd / pair_bwd mutually inverse, mask bit k <=> pair[k] >= 0,
  masks ascending, argsort a permutation, row-major copies equal the tables;
* gather-GEMM: linearity in the features, and the adjoint identities
  <conv(x), g> == <x, dgrad(g)> == <W, wgrad(x, g)> (fp32 reductions of the
  fp16 results, tolerance 2e-3 relative as specified for fp16);
* pooling: max pool is idempotent under re-scaling by a positive constant and
  never negative; avg pool of a constant field is that constant.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _scene(batch, n_range, seed=5):
    from spconv_triton_b200.scenes import lidar_like_batch

    return torch.from_numpy(lidar_like_batch(seed, batch, n_range)).to(DEV)


def _lin(indices, shape):
    lin = indices[:, 0].long()
    for i, s in enumerate(shape):
        lin = lin * int(s) + indices[:, i + 1].long()
    return lin


def _check_rulebook(res, n_in, out_shape, subm):
    out_inds, npl, pf, pb, pmf, pmb, maf, mab, masks = res
    kv, n_out = pf.shape
    if not subm:
        lin = _lin(out_inds, out_shape)
        assert bool((lin[1:] > lin[:-1]).all()), "output coordinates are not strictly ascending"
    # pair_fwd and pair_bwd are inverse maps
    k_idx = torch.arange(kv, device=DEV)[:, None].expand(kv, n_out)
    valid = pf >= 0
    assert int(valid.sum()) == int((pb >= 0).sum())
    rows = torch.arange(n_out, device=DEV, dtype=torch.int32)[None, :].expand(kv, n_out)
    assert torch.equal(pb[k_idx[valid], pf[valid].long()], rows[valid])
    # masks
    for table, pm, ma in ((pf, pmf, maf),) + (((pb, pmb, mab),) if pmb else ()):
        n = table.shape[1]
        bits = torch.zeros(n, dtype=torch.int64, device=DEV)
        for k in range(kv):
            bits |= (table[k] >= 0).long() << k
        m = pm[0][:, 0].long() & 0xFFFFFFFF
        a = ma[0].long()
        assert bool((m[1:] >= m[:-1]).all()), "masks not ascending"
        assert torch.equal(torch.sort(a).values, torch.arange(n, device=DEV)), "argsort is not a permutation"
        assert torch.equal(m, bits[a])
        # stable: equal masks keep ascending row order
        same = m[1:] == m[:-1]
        assert bool((a[1:][same] > a[:-1][same]).all())
    rm = pf._spc_rowmajor
    assert torch.equal(rm[:, :kv].t().contiguous(), pf) and bool((rm[:, kv:] == -1).all())
    return int(valid.sum())


def test_config2_strided_conv_64_128_fp16():
    """BASELINE configs[1]: SparseConv3d k3 s2 p1, 64 -> 128, fp16, batch 4, ~120k voxels/sample."""
    from spconv_triton_b200.pytorch._impl import gemm as G
    from spconv_triton_b200.pytorch._impl import pairs as P

    shape, batch = [41, 1600, 1408], 4
    idx = _scene(batch, (120000, 120000))
    n_in = idx.shape[0]
    out_shape = P.get_conv_output_size(shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3)
    assert out_shape == [21, 800, 704]
    res = P.igemm_pairs(idx, batch, shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, True, False)
    n_pairs = _check_rulebook(res, n_in, out_shape, False)
    out_inds, _, pf, pb, pmf, pmb, maf, mab, _ = res
    n_out = out_inds.shape[0]
    assert n_out > n_in and n_pairs >= n_out  # LiDAR-like scenes dilate under k3 s2
    gen = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(n_in, 64, device=DEV, generator=gen).half()
    y = torch.randn(n_in, 64, device=DEV, generator=gen).half()
    w = (torch.randn(128, 27, 64, device=DEV, generator=gen) / (27 * 64) ** 0.5).half()
    g = torch.randn(n_out, 128, device=DEV, generator=gen).half()
    kw = dict(pair_mask=pmf[0][:, 0], mask_argsort=maf[0])
    fx = G.conv_forward(x, w, pf, n_out, **kw).float()
    fy = G.conv_forward(y, w, pf, n_out, **kw).float()
    fxy = G.conv_forward((x.float() * 0.5 + y.float() * 0.25).half(), w, pf, n_out, **kw).float()
    lin_err = (fxy - (0.5 * fx + 0.25 * fy)).abs().max() / fx.abs().max()
    assert lin_err.item() <= 4e-3, f"linearity {lin_err.item():.2e}"
    din = G.conv_backward_input(g, w, pb, n_in, pair_mask=pmb[0][:, 0], mask_argsort=mab[0]).float()
    dw = G.conv_backward_weight(x, g, pf, (128, 27, 64)).float()
    a = (fx.double() * g.double()).sum()
    b = (x.double() * din.double()).sum()
    c = (w.double() * dw.double()).sum()
    scale = (fx.double().abs() * g.double().abs()).sum()
    assert abs(a - b).item() <= 2e-3 * scale.item() and abs(a - c).item() <= 2e-3 * scale.item()
    G.check_device_status()


def test_config3_backbone_rulebooks_and_determinism():
    """BASELINE configs[2]: the VoxelNet-style backbone, batch 8, 16k-24k voxels/sample."""
    import bench
    import spconv_triton_b200.pytorch as sp

    idx = _scene(8, (16000, 24000), seed=11)
    feats = torch.rand(idx.shape[0], 4, device=DEV).half()
    net = bench.init_backbone(bench.build_backbone()).half().eval().to(DEV)
    with torch.no_grad():
        a = net(sp.SparseConvTensor(feats, idx, bench.GRID, 8))
        b = net(sp.SparseConvTensor(feats, idx, bench.GRID, 8))
    assert torch.equal(a.indices, b.indices) and torch.equal(a.features, b.features)
    assert a.spatial_shape == [6, 200, 176] and bool(torch.isfinite(a.features).all())
    assert float(a.features.min()) >= 0.0  # ends with ReLU
    shape = bench.GRID
    for key, d in a.indice_dict.items():
        res = (d.out_indices, None, d.pair_fwd, d.pair_bwd if d.pair_bwd.numel() else None, d.pair_mask_fwd_splits,
               d.pair_mask_bwd_splits, d.mask_argsort_fwd_splits, d.mask_argsort_bwd_splits, d.masks)
        if d.is_subm:
            # eval-mode subm rulebooks carry no pair_bwd: check fwd against its own mirror
            pf = d.pair_fwd
            kv = pf.shape[0]
            valid = pf >= 0
            k_idx = torch.arange(kv, device=DEV)[:, None].expand_as(pf)
            rows = torch.arange(pf.shape[1], device=DEV, dtype=torch.int32)[None, :].expand_as(pf)
            assert torch.equal(pf[(kv - 1 - k_idx)[valid], pf[valid].long()], rows[valid])
            assert torch.equal(pf[kv // 2], torch.arange(pf.shape[1], device=DEV, dtype=torch.int32))
        else:
            _check_rulebook(res, d.indices.shape[0], d.out_spatial_shape, False)


def test_config5_pools_256_channels():
    """BASELINE configs[4]: SparseMaxPool3d k2 s2 and SparseAvgPool3d k3 s1 at C = 256 on ~30 %-occupancy blobs."""
    import spconv_triton_b200.pytorch as sp

    rng = np.random.default_rng(3)
    grid, batch, n = [128, 128, 128], 2, 200000
    rows = []
    for b in range(batch):
        centres = rng.integers(16, 112, size=(40, 3))
        pts = np.concatenate([c + np.rint(rng.standard_normal((9000, 3)) * 6) for c in centres]).astype(np.int64)
        pts = np.clip(pts, 0, 127)
        pts = np.unique(pts, axis=0)
        pts = pts[rng.permutation(pts.shape[0])[:n]]
        rows.append(np.concatenate([np.full((pts.shape[0], 1), b), pts], 1))
    idx = torch.from_numpy(np.concatenate(rows).astype(np.int32)).to(DEV)
    feats = torch.randn(idx.shape[0], 256, device=DEV).half()
    x = sp.SparseConvTensor(feats, idx, grid, batch)
    mp = sp.SparseMaxPool3d(2, 2)
    out = mp(x)
    assert float(out.features.min()) >= 0.0
    out2 = mp(sp.SparseConvTensor(feats * 2, idx, grid, batch))
    assert torch.equal(out2.features, out.features * 2)  # exact: scaling by two commutes with max(0, .)
    ap = sp.SparseAvgPool3d(3, 1)
    const = ap(sp.SparseConvTensor(torch.full_like(feats, 0.75), idx, grid, batch))
    assert torch.equal(const.features, torch.full_like(const.features, 0.75))
    assert const.indices.shape[0] > idx.shape[0]  # k3 s1 p0 dilates
