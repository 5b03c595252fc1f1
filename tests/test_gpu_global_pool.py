"""Global max / average pooling on CUDA (through the C ABI) against outputs and gradients of the
reference's modules (tests/golden/ref_gpool.pt) and against torch on larger seeded inputs."""

from pathlib import Path

import pytest
import torch

GOLD = torch.load(Path(__file__).parent / "golden" / "ref_gpool.pt", weights_only=False)["cases"]
# mean: fp64 accumulation here, fp32 in torch; compared after rounding to the feature dtype
MEAN_TOL = {torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}


def module(is_mean):
    import spconv_triton_b200.pytorch as sp

    return sp.SparseGlobalAvgPool() if is_mean else sp.SparseGlobalMaxPool()


@pytest.mark.gpu
@pytest.mark.parametrize("case", GOLD, ids=lambda c: c["id"])
def test_reference_vectors(case):
    import spconv_triton_b200.pytorch as sp

    dtype = case["features"].dtype
    feats = case["features"].cuda().requires_grad_(True)
    x = sp.SparseConvTensor(feats, case["indices"].cuda(), [64, 64, 64], case["batch_size"])
    out = module(case["is_mean"])(x)
    assert out.shape == case["expect_out"].shape and out.dtype == dtype
    (out.float() * case["weight"].cuda()).sum().backward()
    if case["is_mean"]:
        tol = MEAN_TOL[dtype]
        torch.testing.assert_close(out.float().cpu(), case["expect_out"], rtol=tol, atol=tol)
        torch.testing.assert_close(feats.grad.float().cpu(), case["expect_grad"], rtol=tol, atol=tol * 1e-2)
    else:
        assert torch.equal(out.float().cpu(), case["expect_out"])           # bit-exact maxima
        torch.testing.assert_close(feats.grad.float().cpu(), case["expect_grad"], rtol=MEAN_TOL[dtype], atol=0)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("channels", [1, 64, 200])
def test_large_against_torch(dtype, channels):
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(3)
    n, batch = 300_000, 6
    feats = torch.randn(n, channels, generator=g).to(dtype).cuda()
    b = torch.randint(0, batch, (n,), generator=g)
    for order in ("sorted", "shuffled"):
        bb = (torch.sort(b).values if order == "sorted" else b).cuda()
        idx = torch.cat([bb[:, None], torch.zeros(n, 3, dtype=torch.int64, device="cuda")], 1).int()
        x = sp.SparseConvTensor(feats, idx, [8, 8, 8], batch)
        got_max, got_mean = module(False)(x), module(True)(x)
        for s in range(batch):
            rows = feats[bb == s]
            assert torch.equal(got_max[s], rows.max(0).values)
            want = rows[:, 0].double().mean()
            assert abs(float(got_mean[s]) - float(want)) <= MEAN_TOL[dtype] * max(1.0, abs(float(want)))


@pytest.mark.gpu
def test_nan_and_empty_sample():
    import spconv_triton_b200.pytorch as sp

    feats = torch.tensor([[1.0, 2.0], [float("nan"), -1.0], [3.0, 0.5]]).cuda()
    idx = torch.tensor([[0, 0, 0, 0], [0, 1, 0, 0], [0, 2, 0, 0]], dtype=torch.int32).cuda()
    out = module(False)(sp.SparseConvTensor(feats, idx, [4, 4, 4], 1))
    assert torch.isnan(out[0, 0]) and float(out[0, 1]) == 2.0                # NaN propagates like torch.max
    x2 = sp.SparseConvTensor(feats, idx, [4, 4, 4], 2)                        # sample 1 has no rows
    with pytest.raises(RuntimeError):
        module(False)(x2)
    mean = module(True)(x2)
    assert torch.isnan(mean[0]) and torch.isnan(mean[1])                      # NaN input; 0 / 0


def test_cpu_is_refused():
    import spconv_triton_b200.pytorch as sp

    x = sp.SparseConvTensor(torch.zeros(2, 3), torch.zeros(2, 4, dtype=torch.int32), [4, 4, 4], 1)
    with pytest.raises(NotImplementedError):
        module(True)(x)
