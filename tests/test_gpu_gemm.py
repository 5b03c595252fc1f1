"""Gather-GEMM parity on the GPU through the C ABI: forward, input gradient
and weight gradient against the reference's vectors and against the CPU
oracle (fp64 accumulation).  Tolerances are the ones the hot path is specified
to, measured against the largest reference magnitude: 1e-5 relative for fp32
(IEEE mode) and 2e-3 for fp16/bf16 (bf16 has 3 fewer mantissa bits than fp16,
so its output rounding alone is 4e-3).  TF32 is held to 1e-3 of the fp64 oracle
here (its operands carry 10 mantissa bits); test_gpu_config_parity.py compares
it with fp64 arithmetic on the TF32-rounded operands at 1e-5."""

import numpy as np
import pytest
import torch

from conftest import feature_case_names
from gpu_util import DEV, rel_err, to_np, unique_coords
from oracle import features as of
from oracle import rulebook as orb

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-5, "float16": 2e-3, "bfloat16": 8e-3, "tf32": 1e-3}
GEMM_CASES = [n for n in feature_case_names() if not n.startswith(("max", "avg"))]


def _gemm():
    from spconv_triton_b200.pytorch._impl import gemm

    return gemm


@pytest.fixture(params=["simt", "cpasync", "auto"])
def gemm_path(request):
    from spconv_triton_b200 import _lib

    g = _gemm()
    old = g.GEMM_PATH
    # "cpasync": like auto, but the tcgen05 kernels are fed by cp.async, never by TMA
    g.GEMM_PATH = {"simt": _lib.SPC_GEMM_SIMT, "auto": _lib.SPC_GEMM_AUTO,
                   "cpasync": _lib.SPC_GEMM_TCGEN05_CPASYNC}[request.param]
    yield request.param
    g.GEMM_PATH = old
    g.check_device_status()  # no tcgen05 kernel may have given up on a wait


@pytest.mark.parametrize("name", GEMM_CASES)
def test_matches_reference_vectors(ref_ops, name, gemm_path):
    spec = ref_ops.features[name]
    rb, dt = spec["rulebook"], spec["dtype"]
    g = lambda k: torch.from_numpy(ref_ops.get(f"ft/{name}/{k}"))  # noqa: E731
    pf = torch.from_numpy(ref_ops.rb(rb, "ig_pair_fwd")).to(DEV)
    pb = torch.from_numpy(ref_ops.rb(rb, "ig_pair_bwd")).to(DEV)
    feats, w, gout = g("features").to(DEV), g("weight").to(DEV), g("grad_out").to(DEV)
    bias = g("bias").to(DEV) if ref_ops.has(f"ft/{name}/bias") else None
    kv = pf.shape[0]
    pm = ma = None
    if kv <= 32:
        pm = torch.from_numpy(ref_ops.rb(rb, "ig_pm_fwd0")).to(DEV)[:, 0]
        ma = torch.from_numpy(ref_ops.rb(rb, "ig_ma_fwd0")).to(DEV)
    G = _gemm()
    out = G.conv_forward(feats, w, pf, pf.shape[1], bias=bias, pair_mask=pm, mask_argsort=ma)
    din = G.conv_backward_input(gout, w, pb, feats.shape[0])
    dw = G.conv_backward_weight(feats, gout, pf, tuple(w.shape))
    assert out.dtype == feats.dtype and din.dtype == gout.dtype and dw.dtype == gout.dtype
    assert rel_err(to_np(out.float()), g("out").float().numpy()) <= TOL[dt]
    assert rel_err(to_np(din.float()), g("din").float().numpy()) <= TOL[dt]
    assert rel_err(to_np(dw.float()), g("dw").float().numpy()) <= TOL[dt]


SHAPES = [
    # (c_in, c_out, dtype, subm, kv-geometry)
    (16, 16, torch.float32, True),
    (4, 16, torch.float16, True),
    (16, 32, torch.float16, False),
    (32, 32, torch.float16, True),
    (64, 64, torch.float16, True),
    (64, 128, torch.float16, False),
    (128, 64, torch.bfloat16, False),
    (48, 80, torch.float16, True),
    (24, 40, torch.float32, False),
    (256, 256, torch.float16, True),
    (136, 130, torch.float16, True),
    # thin layers (one thread per output row): odd widths, every dtype, strided
    (3, 8, torch.float32, True),
    (5, 20, torch.bfloat16, False),
    (8, 32, torch.float16, False),
    (1, 1, torch.float32, True),
]


def _scene(seed, subm, n=12000):
    shape, batch = [24, 40, 36], 2
    idx_np = unique_coords(seed, n, batch, shape)
    if subm:
        res = orb.igemm_pairs(idx_np, batch, shape, [3] * 3, [1] * 3, [1] * 3, [1] * 3, [0] * 3, True, False, True, False)
    else:
        res = orb.igemm_pairs(idx_np, batch, shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, True, False)
    return idx_np, res


@pytest.mark.parametrize("case", range(len(SHAPES)))
def test_matches_oracle(case, gemm_path):
    c_in, c_out, dtype, subm = SHAPES[case]
    idx_np, res = _scene(900 + case, subm)
    _, _, pf, pb, pmf, pmb, maf, mab, _ = res
    n_in, n_out, kv = idx_np.shape[0], pf.shape[1], pf.shape[0]
    gen = torch.Generator().manual_seed(case)
    feats = torch.randn(n_in, c_in, generator=gen).to(dtype)
    w = (torch.randn(c_out, kv, c_in, generator=gen) / (kv * c_in) ** 0.5).to(dtype)
    bias = torch.randn(c_out, generator=gen).to(dtype)
    gout = torch.randn(n_out, c_out, generator=gen).to(dtype)
    G = _gemm()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    out = G.conv_forward(feats.to(DEV), w.to(DEV), d(pf), n_out, bias=bias.to(DEV), pair_mask=d(pmf[0])[:, 0],
                         mask_argsort=d(maf[0]))
    bwd_mask = dict(pair_mask=d(pmb[0])[:, 0], mask_argsort=d(mab[0])) if pmb else {}
    din = G.conv_backward_input(gout.to(DEV), w.to(DEV), d(pb), n_in, **bwd_mask)
    dw = G.conv_backward_weight(feats.to(DEV), gout.to(DEV), d(pf), (c_out, kv, c_in))
    tol = TOL[str(dtype).split(".")[1]]
    e_out = of.conv_forward(feats, w, pf, n_out, bias=bias, out_dtype=torch.float64)
    e_din = of.conv_backward_input(gout.double(), w, pb, n_in)
    e_dw = of.conv_backward_weight(feats, gout.double(), pf, (c_out, kv, c_in))
    assert rel_err(to_np(out.double()), e_out.numpy()) <= tol, "forward"
    assert rel_err(to_np(din.double()), e_din.numpy()) <= tol, "dgrad"
    assert rel_err(to_np(dw.double()), e_dw.numpy()) <= tol, "wgrad"


def test_tf32_switch_is_live(gemm_path):
    """fp32 inputs use IEEE arithmetic unless constants.SPCONV_ALLOW_TF32 is set
    at call time; TF32 results stay within 1e-3 of the fp64 oracle but are not
    as close as IEEE (reference: _impl/gemm.py:460-463)."""
    from spconv_triton_b200 import constants

    idx_np, res = _scene(4242, True)
    pf, pmf, maf = res[2], res[4], res[6]
    n, kv, c = idx_np.shape[0], pf.shape[0], 64
    gen = torch.Generator().manual_seed(7)
    feats = torch.randn(n, c, generator=gen)
    w = torch.randn(c, kv, c, generator=gen) / (kv * c) ** 0.5
    G = _gemm()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    e = of.conv_forward(feats, w, pf, n, out_dtype=torch.float64).numpy()
    ieee = G.conv_forward(feats.to(DEV), w.to(DEV), d(pf), n, mask_argsort=d(maf[0]), pair_mask=d(pmf[0])[:, 0])
    assert rel_err(to_np(ieee.double()), e) <= TOL["float32"]
    constants.SPCONV_ALLOW_TF32 = True
    try:
        tf32 = G.conv_forward(feats.to(DEV), w.to(DEV), d(pf), n, mask_argsort=d(maf[0]), pair_mask=d(pmf[0])[:, 0])
    finally:
        constants.SPCONV_ALLOW_TF32 = False
    assert rel_err(to_np(tf32.double()), e) <= TOL["tf32"]


def test_out_dtype_and_empty(gemm_path):
    idx_np, res = _scene(11, True, n=500)
    pf = res[2]
    n, kv = idx_np.shape[0], pf.shape[0]
    feats = torch.randn(n, 16).half().to(DEV)
    w = torch.randn(16, kv, 16).half().to(DEV) * 0.1
    G = _gemm()
    out = G.conv_forward(feats, w, torch.from_numpy(pf).to(DEV), n, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    e = of.conv_forward(feats.cpu(), w.cpu(), pf, n, out_dtype=torch.float64).numpy()
    assert rel_err(to_np(out.double()), e) <= 1e-5 * 10  # fp16 inputs, fp32 accumulate and output
    empty = G.conv_forward(feats, w, torch.from_numpy(pf[:, :0].copy()).to(DEV), 0)
    assert tuple(empty.shape) == (0, 16)


def test_deterministic(gemm_path):
    idx_np, res = _scene(3, False)
    pf, pb = res[2], res[3]
    n_in, n_out, kv = idx_np.shape[0], pf.shape[1], pf.shape[0]
    feats = torch.randn(n_in, 32).half().to(DEV)
    w = (torch.randn(64, kv, 32) * 0.05).half().to(DEV)
    gout = torch.randn(n_out, 64).half().to(DEV)
    G = _gemm()
    pfd, pbd = torch.from_numpy(pf).to(DEV), torch.from_numpy(pb).to(DEV)
    for fn in (lambda: G.conv_forward(feats, w, pfd, n_out), lambda: G.conv_backward_input(gout, w, pbd, n_in),
               lambda: G.conv_backward_weight(feats, gout, pfd, (64, kv, 32))):
        assert torch.equal(fn(), fn())


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("c_in,c_out", [(32, 64), (4, 16), (20, 12)])
def test_residual_added_in_the_store(gemm_path, dtype, c_in, c_out):
    """out = conv(x) + residual in one pass (every forward kernel), against the fp64 oracle plus the
    residual; and through the layer: add_input in training mode gives the same output and the same
    gradients as the separate addition."""
    idx_np, res = _scene(77, True)
    pf, pmf, maf = res[2], res[4], res[6]
    n, kv = idx_np.shape[0], pf.shape[0]
    gen = torch.Generator().manual_seed(5)
    feats = torch.randn(n, c_in, generator=gen).to(dtype)
    w = (torch.randn(c_out, kv, c_in, generator=gen) / (kv * c_in) ** 0.5).to(dtype)
    resid = torch.randn(n, c_out, generator=gen).to(dtype)
    G = _gemm()
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)  # noqa: E731
    out = G.conv_forward(feats.to(DEV), w.to(DEV), d(pf), n, mask_argsort=d(maf[0]), pair_mask=d(pmf[0])[:, 0],
                         residual=resid.to(DEV))
    e = of.conv_forward(feats, w, pf, n, out_dtype=torch.float64) + resid.double()
    assert rel_err(to_np(out.double()), e.numpy()) <= TOL[str(dtype).split(".")[-1]]


def test_add_input_in_training_is_fused_and_differentiable():
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.pytorch import ops

    idx_np, _ = _scene(78, True, n=3000)
    idx = torch.from_numpy(idx_np).to(DEV)
    n = idx_np.shape[0]
    torch.manual_seed(2)
    conv = sp.SubMConv3d(16, 32, 3, padding=1, bias=False, indice_key="a").to(DEV).train()
    x0 = torch.randn(n, 16, device=DEV)
    r0 = torch.randn(n, 32, device=DEV)
    shape, batch = [24, 40, 36], 2  # the grid _scene draws from
    seen = []
    orig = ops.implicit_gemm

    def spy(*a, **kw):
        seen.append(kw.get("_residual") is not None)
        return orig(*a, **kw)

    ops.implicit_gemm = spy
    try:
        xa, ra = x0.clone().requires_grad_(True), r0.clone().requires_grad_(True)
        ya = conv(sp.SparseConvTensor(xa, idx, shape, batch), add_input=sp.SparseConvTensor(ra, idx, shape, batch))
        ya.features.pow(2).sum().backward()
    finally:
        ops.implicit_gemm = orig
    assert seen == [True]  # the residual went into the kernel
    ga, gra, gwa = xa.grad.clone(), ra.grad.clone(), conv.weight.grad.clone()
    conv.weight.grad = None
    xb, rb = x0.clone().requires_grad_(True), r0.clone().requires_grad_(True)
    yb = conv(sp.SparseConvTensor(xb, idx, shape, batch))
    fb = yb.features + rb
    fb.pow(2).sum().backward()
    assert rel_err(to_np(ya.features), to_np(fb)) <= 1e-5
    assert rel_err(to_np(ga), to_np(xb.grad)) <= 1e-5
    assert rel_err(to_np(gra), to_np(rb.grad)) <= 1e-5
    assert rel_err(to_np(gwa), to_np(conv.weight.grad)) <= 1e-5
