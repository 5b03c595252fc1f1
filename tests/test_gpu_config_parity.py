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
* fp32        TF32 mode against fp64 of the TF32-rounded operands (1e-5: the same
              arithmetic as the reference's tl.dot) with the distance to plain fp64
              measured beside it; IEEE mode (split operands on the tensor cores) 1e-5.

Tolerances (relative to the largest magnitude of the expected tensor):
fp16 2e-3, fp32 1e-5.  Indices and rulebooks: bit-exact.
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
    # half of the points uniform in the grid, half in a dense corner so that neighbours exist in
    # four dimensions; coordinates are unique (uniform points that fall into the corner are dropped)
    rng = np.random.default_rng(2)
    far = uniform_batch(9, 1, n, tuple(shape))
    far = far[(far[:, 1:] >= 14).any(axis=1)][: n - n // 2]
    corner = np.stack(np.unravel_index(rng.choice(14 ** 4, n // 2, replace=False), [14] * 4), 1).astype(np.int32)
    corner = np.concatenate([np.zeros((n // 2, 1), np.int32), corner], 1)
    idx_np = np.concatenate([far, corner], 0)
    idx_np = np.ascontiguousarray(idx_np[rng.permutation(idx_np.shape[0])])
    n = idx_np.shape[0]
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
    """Encoder / decoder at ~110k voxels under fp16 autocast, training mode.

    Forward: the whole network against the same network in fp64 on the CPU over the oracle's
    tables (tolerance 1e-2: fp16 activations through fifteen layers with batch statistics).
    Backward: layer by layer.  ReLU makes the gradient of the whole network a discontinuous
    function of the activations (a unit whose fp16 pre-activation has the other sign than its fp64
    value switches its whole path), so the end-to-end gradient is no parity measure; instead every
    convolution's input gradient and weight gradient, as autograd produced them inside the module
    stack, are compared with fp64 sums over the oracle's tables evaluated on the very tensors that
    layer saw (its fp16 input features and the fp16 gradient of its output), at the fp16 tolerance
    2e-3.  That covers the table roles of strided and inverse layers, the autocast casts and the
    bias-free training path."""
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

    # ---- the oracle's tables for every indice_key ----------------------------------------------
    three = lambda v: [v] * 3  # noqa: E731
    tabs, cur_idx, cur_shape = {}, idx_np, grid
    tabs["subm0"] = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(1), three(1), three(1), three(0),
                                    True, False, True, False)
    for lvl in range(1, len(widths)):
        r = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(2), three(1), three(1), three(0), False, False,
                            True, False)
        tabs[f"down{lvl}"] = r
        cur_idx, cur_shape = r[0], orb.conv_output_size(cur_shape, three(3), three(2), three(1), three(1))
        tabs[f"subm{lvl}"] = orb.igemm_pairs(cur_idx, batch, cur_shape, three(3), three(1), three(1), three(1),
                                             three(0), True, False, True, False)

    def tables_of(m):
        r = tabs[m.indice_key]
        # an inverse layer runs the strided layer's rulebook backwards
        return (r[3], r[2]) if m.inverse else (r[2], r[3])

    # ---- the same network in fp64 on the CPU (forward check) ----------------------------------
    ref_layers, convs = [], []
    for m in net._modules.values():
        if hasattr(m, "weight_shape"):
            w = m.weight.detach().reshape(m.out_channels, -1, m.in_channels)
            ref_layers.append(_GatherMatmul(w, tables_of(m)[0]))
            convs.append(m)
        elif isinstance(m, torch.nn.BatchNorm1d):
            bn = torch.nn.BatchNorm1d(m.num_features, eps=m.eps, momentum=m.momentum).double()
            bn.load_state_dict({k: v.double() if v.is_floating_point() else v for k, v in m.state_dict().items()})
            ref_layers.append(bn)
        else:
            ref_layers.append(torch.nn.ReLU())
    with torch.no_grad():
        y_ref = torch.nn.Sequential(*ref_layers).train()(feats.double())

    # ---- the CUDA path, with every convolution's tensors captured --------------------------------
    seen = {}

    def capture(m, args, output):
        rec = seen.setdefault(id(m), {})
        rec["f_in"] = args[0].features.detach()
        output.features.register_hook(lambda g, rec=rec: rec.__setitem__("g_out", g.detach()))
        if args[0].features.requires_grad:
            args[0].features.register_hook(lambda g, rec=rec: rec.__setitem__("g_in", g.detach()))

    handles = [m.register_forward_hook(capture) for m in convs]
    net = net.to(DEV).train()
    x = feats.to(DEV).requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        out = net(sp.SparseConvTensor(x, torch.from_numpy(idx_np).to(DEV), grid, batch))
        loss = out.features.float().pow(2).sum() / 128.0
    loss.backward()
    torch.cuda.synchronize()
    for h in handles:
        h.remove()
    assert out.features.dtype == torch.float16
    np.testing.assert_array_equal(to_np(out.indices), idx_np)
    errs = {"forward (whole network)": (rel_err(to_np(out.features.double()), y_ref.numpy()), 1e-2)}
    for i, m in enumerate(convs):
        rec = seen[id(m)]
        kind = "inverse" if m.inverse else ("subm" if m.subm else "strided")
        name = f"layer {i} ({kind} {m.in_channels}->{m.out_channels}, {m.indice_key})"
        f_in = rec["f_in"].half().cpu().double()     # what the autocast forward fed the kernel
        g_out = rec["g_out"].half().cpu().double()
        w = m.weight.detach().half().cpu().double().reshape(m.out_channels, -1, m.in_channels)
        t_fwd, t_bwd = tables_of(m)
        e_dw = of.conv_backward_weight(f_in, g_out, t_fwd, tuple(w.shape))
        errs[name + " weight gradient"] = (rel_err(to_np(m.weight.grad.double().reshape(w.shape)), e_dw.numpy()), 2e-3)
        e_din = of.conv_backward_input(g_out, w, t_bwd, f_in.shape[0])
        errs[name + " input gradient"] = (rel_err(to_np(rec["g_in"].double()), e_din.numpy()), 2e-3)
    report = "\n".join(f"  {k}: {v:.2e} (limit {lim:.0e})" for k, (v, lim) in errs.items())
    print("UNet forward + backward under autocast against fp64:\n" + report)
    bad = [k for k, (v, lim) in errs.items() if not v <= lim]
    assert not bad, f"beyond tolerance: {bad}\n{report}"


# ---------------------------------------------------------------------------------------------
# fp32 layers: TF32 mode and IEEE mode, both on the tensor cores
# ---------------------------------------------------------------------------------------------
def _rna_tf32(t):
    """Round fp32 to the nearest TF32 number, ties away from zero (what cvt.rna.tf32.f32 and the
    reference's tl.dot(input_precision="tf32") do to an operand)."""
    bits = t.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    bits = ((bits + 0x1000) & 0xFFFFE000) & 0xFFFFFFFF
    bits = torch.where(bits >= 2 ** 31, bits - 2 ** 32, bits).to(torch.int32)
    return bits.view(torch.float32)


@pytest.mark.parametrize("c_in,c_out", [(32, 32), (64, 128), (128, 64), (16, 16)])
def test_fp32_layers_on_tensor_cores(c_in, c_out):
    """Features ~ N(0,1), weights ~ N(0, 1/(kv*c_in)).

    TF32 mode (SPCONV_ALLOW_TF32): operands are rounded to TF32 (10-bit mantissa, round to nearest)
    and multiplied exactly with fp32 accumulation, like the reference's tl.dot.  Against an fp64
    evaluation of the SAME rounded operands the result must agree to 1e-5 (only the accumulation
    differs); against fp64 of the unrounded operands the operand rounding itself (2^-11 per factor)
    shows: that distance is measured, printed and held below 1e-3 -- no single-pass TF32 product,
    the reference's included, can be closer.

    IEEE mode (the default) must hold the fp32 tolerance 1e-5 against fp64: short reductions run
    split operands on the tensor cores, long ones (whose tensor-core accumulation error would
    exceed it) the IEEE kernels on the CUDA cores."""
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

    def expected(f, wt, go):
        return (of.conv_forward(f.double(), wt.double(), to_np(pf), n, out_dtype=torch.float64),
                of.conv_backward_input(go.double(), wt.double(), to_np(pb), n))

    def run():
        fwd = G.conv_forward(feats.to(DEV), w.to(DEV), pf, n, mask_argsort=res[6][0], pair_mask=res[4][0])
        din = G.conv_backward_input(gout.to(DEV), w.to(DEV), pb, n)
        G.check_device_status()
        return fwd, din

    launches = G._lib.load().spc_launch_count
    exact = expected(feats, w, gout)
    old = constants.SPCONV_ALLOW_TF32
    try:
        constants.SPCONV_ALLOW_TF32 = True
        got = run()
        rounded = expected(_rna_tf32(feats), _rna_tf32(w), _rna_tf32(gout))
        for name, a, e_same, e_exact in zip(("forward", "input gradient"), got, rounded, exact):
            same = rel_err(to_np(a.double()), e_same.numpy())
            dist = rel_err(to_np(a.double()), e_exact.numpy())
            print(f"TF32 {c_in}->{c_out} {name}: {same:.2e} against fp64 of the rounded operands, "
                  f"{dist:.2e} against fp64 of the fp32 operands")
            assert same <= 1e-5, f"TF32 {name} {c_in}->{c_out}: {same:.2e} beyond the accumulation error"
            assert dist <= 1e-3, f"TF32 {name} {c_in}->{c_out}: {dist:.2e}"
        constants.SPCONV_ALLOW_TF32 = False
        got = run()
        for name, a, e in zip(("forward", "input gradient"), got, exact):
            err = rel_err(to_np(a.double()), e.numpy())
            print(f"fp32 IEEE mode {c_in}->{c_out} {name}: {err:.2e}")
            assert err <= 1e-5, f"fp32 {name} {c_in}->{c_out}: {err:.2e} > 1e-5"
        # and the CUDA-core IEEE kernels behind the switch
        G.FP32_ON_TENSOR_CORES = False
        got = run()
        for name, a, e in zip(("forward", "input gradient"), got, exact):
            assert rel_err(to_np(a.double()), e.numpy()) <= 1e-5
    finally:
        constants.SPCONV_ALLOW_TF32 = old
        G.FP32_ON_TENSOR_CORES = True
    assert launches() > 0
