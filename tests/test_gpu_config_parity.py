"""Parity with the CPU oracle AT the benchmark configurations, through the
module API (the composition of rulebook, GEMM, fused epilogue, run-ahead and
autograd), at sizes the oracle finishes in seconds:

* configs[2]  the VoxelNet-style backbone of bench.py on one ~20k-voxel sample,
              BatchNorm/ReLU fold and rulebook run-ahead on and off;
* configs[4]  SubMConv3d k5 256 -> 256 (kv 125, Native rulebook) on 120k blob
              voxels, SubMConv4d k3 64 -> 64 on 50k voxels;
* configs[3]  encoder / decoder with SparseInverseConv3d reusing the encoder's
              rulebook, forward + backward under fp16 autocast, gradients
              against an fp64 gather-matmul over the oracle's tables;
* TF32        the achieved error of the TF32 path is measured and held at the
              1e-4 the specification names.

Tolerances (relative to the largest magnitude of the expected tensor):
fp16 2e-3, TF32 1e-4, fp32 1e-5.  Indices and rulebooks: bit-exact.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import rel_err, to_np
from oracle import features as of
from oracle import rulebook as orb
from oracle.backbone import run_backbone

pytestmark = pytest.mark.gpu
DEV = "cuda"


# ---------------------------------------------------------------------------------------------
# configs[2]: the backbone
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("fold", [True, False])
@pytest.mark.parametrize("runahead", [True, False])
def test_config3_backbone_matches_oracle(fold, runahead):
    import bench
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200 import constants

    idx, feats = bench.make_scenes(0, n_scenes=1, batch=1)[0]
    net = bench.init_backbone(bench.build_backbone())
    params = bench.oracle_params(net)
    # the oracle keeps fp16 activations between layers, as the fp16 modules do
    e_idx, e_feats, e_shape = run_backbone(bench.LAYERS, params, idx.numpy(), feats, bench.GRID, 1,
                                           acc_dtype=torch.float64)
    net = net.half().eval().to(DEV)
    old = constants.SPCONV_FOLD_BN_RELU, constants.SPCONV_RULEBOOK_RUNAHEAD
    constants.SPCONV_FOLD_BN_RELU, constants.SPCONV_RULEBOOK_RUNAHEAD = fold, runahead
    try:
        with torch.no_grad():
            out = net(sp.SparseConvTensor(feats.to(DEV), idx.to(DEV), bench.GRID, 1))
        torch.cuda.synchronize()
    finally:
        constants.SPCONV_FOLD_BN_RELU, constants.SPCONV_RULEBOOK_RUNAHEAD = old
    assert list(out.spatial_shape) == list(e_shape)
    np.testing.assert_array_equal(to_np(out.indices), e_idx)
    err = rel_err(to_np(out.features.float()), e_feats.float().numpy())
    assert err <= 2e-3, f"backbone features off by {err:.2e} (fold={fold}, runahead={runahead})"


# ---------------------------------------------------------------------------------------------
# configs[4]: k5 256 -> 256 (Native) and the 4-D layer
# ---------------------------------------------------------------------------------------------
def test_config5_subm_k5_native_120k():
    import bench
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.core import ConvAlgo
    from spconv_triton_b200.pytorch._impl import pairs as P

    shape, n = [128] * 3, 120000
    idx = bench.blob_scene(3, 1, n, grid=128)
    idx_np = idx.numpy()
    k, one, zero, pad = [5] * 3, [1] * 3, [0] * 3, [2] * 3
    e_out, e_pair, e_npl = orb.native_pairs(idx_np, 1, shape, k, one, pad, one, zero, True, False)
    out_inds, pair, npl = P.native_pairs(idx.to(DEV), 1, shape, k, one, pad, one, zero, True, False)
    np.testing.assert_array_equal(to_np(pair), e_pair)
    np.testing.assert_array_equal(to_np(npl), e_npl)
    e_pf, e_pb = orb.native_pair_to_tables(e_pair, n, n, False)
    pf, pb = P.native_pair_to_tables(pair, npl, n, n, False)
    np.testing.assert_array_equal(to_np(pf), e_pf)
    np.testing.assert_array_equal(to_np(pb), e_pb)

    # the layer itself: Native is the default algorithm for kv > 32
    torch.manual_seed(0)
    conv = sp.SubMConv3d(256, 256, 5, padding=2, bias=True, indice_key="k5").half().to(DEV)
    assert conv.algo == ConvAlgo.Native
    feats = torch.randn(n, 256).half()
    with torch.no_grad():
        out = conv(sp.SparseConvTensor(feats.to(DEV), idx.to(DEV), shape, 1))
    rows = torch.from_numpy(np.random.default_rng(1).choice(n, 4000, replace=False)).long()
    w = conv.weight.detach().cpu().reshape(256, 125, 256)
    expect = of.conv_forward(feats, w, e_pf[:, rows.numpy()], rows.numel(), bias=conv.bias.detach().cpu(),
                             out_dtype=torch.float64)
    err = rel_err(to_np(out.features[rows.to(DEV)].double()), expect.numpy())
    assert err <= 2e-3, f"k5 256->256 forward off by {err:.2e}"


def test_config5_subm4d_k3_50k():
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.pytorch._impl import pairs as P
    from spconv_triton_b200.scenes import uniform_batch

    shape, n = [64] * 4, 50000
    idx_np = uniform_batch(9, 1, n, tuple(shape))
    # part of the points in a dense corner so that neighbours exist in four dimensions
    rng = np.random.default_rng(2)
    idx_np[: n // 2, 1:] = np.stack(np.unravel_index(rng.choice(14 ** 4, n // 2, replace=False), [14] * 4), 1)
    idx = torch.from_numpy(idx_np)
    k, one, zero = [3] * 4, [1] * 4, [0] * 4
    e_out, e_pair, e_npl = orb.native_pairs(idx_np, 1, shape, k, one, one, one, zero, True, False)
    _, pair, npl = P.native_pairs(idx.to(DEV), 1, shape, k, one, one, one, zero, True, False)
    np.testing.assert_array_equal(to_np(pair), e_pair)
    np.testing.assert_array_equal(to_np(npl), e_npl)
    e_pf, _ = orb.native_pair_to_tables(e_pair, n, n, False)
    assert int((e_pf >= 0).sum()) > 4 * n  # the corner does have neighbours

    torch.manual_seed(0)
    conv = sp.SubMConv4d(64, 64, 3, padding=1, bias=False).half().to(DEV)
    feats = torch.randn(n, 64).half()
    with torch.no_grad():
        out = conv(sp.SparseConvTensor(feats.to(DEV), idx.to(DEV), shape, 1))
    expect = of.conv_forward(feats, conv.weight.detach().cpu().reshape(64, 81, 64), e_pf, n, out_dtype=torch.float64)
    err = rel_err(to_np(out.features.double()), expect.numpy())
    assert err <= 2e-3, f"4-D 64->64 forward off by {err:.2e}"


# ---------------------------------------------------------------------------------------------
# configs[3]: encoder / decoder, forward + backward under autocast
# ---------------------------------------------------------------------------------------------
class _GatherMatmul(torch.nn.Module):
    """fp64 CPU restatement of one sparse convolution over given tables:
    out[m] = sum_k f[pair_fwd[k, m]] @ W[:, k, :]^T, differentiable by torch autograd."""

    def __init__(self, weight, pair_fwd):
        super().__init__()
        self.weight = torch.nn.Parameter(weight.double().clone())
        self.pf = torch.as_tensor(pair_fwd).long()

    def forward(self, f):
        k_out, kv, c_in = self.weight.shape
        out = torch.zeros(self.pf.shape[1], k_out, dtype=torch.float64)
        for k in range(kv):
            col = self.pf[k]
            o = torch.nonzero(col >= 0, as_tuple=True)[0]
            if o.numel():
                out = out.index_add(0, o, f.index_select(0, col[o]) @ self.weight[:, k, :].t())
        return out


def test_config4_unet_forward_backward_autocast():
    import bench
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.scenes import indoor_like_batch

    grid, batch = [512, 512, 64], 2
    idx_np = indoor_like_batch(11, batch, (50000, 60000), tuple(grid))
    n = idx_np.shape[0]
    torch.manual_seed(5)
    feats = torch.rand(n, 4)
    widths = (16, 32, 64)
    net = bench.build_unet(4, widths)
    with torch.no_grad():
        for m in net.modules():
            if hasattr(m, "weight_shape"):  # larger weights than the default init: gradients well above fp16 noise
                fan_in = int(np.prod(m.weight_shape[1:]))
                m.weight.copy_(torch.randn(m.weight_shape) * (2.0 / fan_in) ** 0.5)

    # ---- oracle: the same network in fp64 on the CPU over the oracle's tables -----------------
    three = lambda v: [v] * 3  # noqa: E731
    tabs, cur_idx, cur_shape = {}, idx_np, grid
    levels = len(widths)
    tabs["subm0"] = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(1), three(1), three(1), three(0),
                                    True, False, True, False)
    for lvl in range(1, levels):
        r = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(2), three(1), three(1), three(0), False, False,
                            True, False)
        tabs[f"down{lvl}"] = r
        cur_idx, cur_shape = r[0], orb.conv_output_size(cur_shape, three(3), three(2), three(1), three(1))
        tabs[f"subm{lvl}"] = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(1), three(1), three(1),
                                             three(0), True, False, True, False)
    ref_layers, convs = [], []
    for m in net._modules.values():
        if hasattr(m, "weight_shape"):
            r = tabs[m.indice_key]
            table = r[3] if m.inverse else r[2]  # an inverse layer runs the strided layer's rulebook backwards
            w = m.weight.detach().reshape(m.out_channels, -1, m.in_channels)
            ref_layers.append(_GatherMatmul(w, table))
            convs.append(m)
        elif isinstance(m, torch.nn.BatchNorm1d):
            bn = torch.nn.BatchNorm1d(m.num_features, eps=m.eps, momentum=m.momentum).double()
            bn.load_state_dict({k: v.double() if v.is_floating_point() else v for k, v in m.state_dict().items()})
            ref_layers.append(bn)
        else:
            ref_layers.append(torch.nn.ReLU())
    ref = torch.nn.Sequential(*ref_layers).train()
    x_ref = feats.double().requires_grad_(True)
    y_ref = ref(x_ref)
    (y_ref.pow(2).mean() * 64.0).backward()

    # ---- the CUDA path -------------------------------------------------------------------------
    net = net.to(DEV).train()
    x = feats.to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        out = net(sp.SparseConvTensor(x, torch.from_numpy(idx_np).to(DEV), grid, batch))
        loss = out.features.float().pow(2).mean() * 64.0
    loss.backward()
    torch.cuda.synchronize()
    assert out.features.dtype == torch.float16
    np.testing.assert_array_equal(to_np(out.indices), idx_np)
    # fp16 activations through 3 * (2 * levels - 1) layers, batch statistics: 2e-3 per GEMM compounds
    tol = 1e-2
    err = rel_err(to_np(out.features.double()), y_ref.detach().numpy())
    assert err <= tol, f"UNet forward off by {err:.2e}"
    err = rel_err(to_np(x.grad.double()), x_ref.grad.numpy())
    assert err <= 2 * tol, f"UNet input gradient off by {err:.2e}"
    ref_convs = [m for m in ref if isinstance(m, _GatherMatmul)]
    for i, (m, r) in enumerate(zip(convs, ref_convs)):
        err = rel_err(to_np(m.weight.grad.double().reshape(r.weight.shape)), r.weight.grad.numpy())
        assert err <= 2 * tol, f"weight gradient of convolution {i} ({m.indice_key}) off by {err:.2e}"


# ---------------------------------------------------------------------------------------------
# TF32 at the specified tolerance
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("c_in,c_out", [(32, 32), (64, 128), (128, 64)])
def test_tf32_error_is_within_1e_4(c_in, c_out):
    """Features ~ N(0,1), weights ~ N(0, 1/(kv*c_in)): the TF32 path (10-bit mantissa operands,
    fp32 accumulation) is measured against fp64 and the result written next to the bound."""
    from gpu_util import unique_coords
    from spconv_triton_b200 import constants
    from spconv_triton_b200.pytorch._impl import gemm as G
    from spconv_triton_b200.pytorch._impl import pairs as P

    shape, batch, n = [24, 40, 40], 2, 30000
    idx_np = unique_coords(31, n, batch, shape)
    three = lambda v: [v] * 3  # noqa: E731
    res = P.igemm_pairs(torch.from_numpy(idx_np).to(DEV), batch, shape, three(3), three(1), three(1), three(1),
                        three(0), True, False, True, False)
    pf, pb = res[2], res[3]
    g = torch.Generator().manual_seed(4)
    feats = torch.randn(n, c_in, generator=g)
    w = torch.randn(c_out, 27, c_in, generator=g) / (27 * c_in) ** 0.5
    gout = torch.randn(n, c_out, generator=g)
    e_fwd = of.conv_forward(feats, w, to_np(pf), n, out_dtype=torch.float64)
    e_din = of.conv_backward_input(gout.double(), w, to_np(pb), n)
    e_dw = of.conv_backward_weight(feats.double(), gout.double(), to_np(pf), (c_out, 27, c_in))
    old = constants.SPCONV_ALLOW_TF32
    constants.SPCONV_ALLOW_TF32 = True
    try:
        fwd = G.conv_forward(feats.to(DEV), w.to(DEV), pf, n, mask_argsort=res[6][0], pair_mask=res[4][0])
        din = G.conv_backward_input(gout.to(DEV), w.to(DEV), pb, n)
        dw = G.conv_backward_weight(feats.to(DEV), gout.to(DEV), pf, (c_out, 27, c_in))
        G.check_device_status()
    finally:
        constants.SPCONV_ALLOW_TF32 = old
    errs = dict(forward=rel_err(to_np(fwd.double()), e_fwd.numpy()),
                input_gradient=rel_err(to_np(din.double()), e_din.numpy()),
                weight_gradient=rel_err(to_np(dw.double()), e_dw.numpy()))
    print(f"TF32 {c_in}->{c_out} achieved relative errors: " + ", ".join(f"{k} {v:.2e}" for k, v in errs.items()))
    for name, err in errs.items():
        assert err <= 1e-4, f"TF32 {name} {c_in}->{c_out}: {err:.2e} > 1e-4"
