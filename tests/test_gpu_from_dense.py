"""SparseConvTensor.from_dense on CUDA (through the C ABI) against torch's to_sparse, which is what
the reference calls (core.py:296-304), and against the reference's frozen golden case."""

from pathlib import Path

import pytest
import torch


def reference_from_dense(x):
    sp = x.to_sparse(x.ndim - 1)
    return sp.values(), sp.indices().permute(1, 0).contiguous().int()


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype", [((2, 8, 9, 10, 16), torch.float32), ((3, 40, 33, 5), torch.float16),
                                         ((1, 50, 3), torch.float64), ((2, 6, 7, 8, 9, 4), torch.bfloat16),
                                         ((4, 100, 88, 1), torch.float32), ((2, 16, 16, 16, 7), torch.int32),
                                         ((2, 12, 12, 3), torch.int64), ((2, 12, 12, 3), torch.uint8)])
def test_matches_to_sparse(shape, dtype):
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(1)
    keep = (torch.rand(shape[:-1], generator=g) < 0.2)[..., None]
    vals = torch.randint(-3, 4, shape, generator=g)                   # zeros inside kept cells too
    x = (vals * keep).to(dtype).cuda()
    if dtype.is_floating_point:
        x.view(-1)[5] = -0.0                                          # negative zero is zero
        x.view(-1)[-1] = float("nan")                                 # NaN is not
    got = sp.SparseConvTensor.from_dense(x)
    want_f, want_i = reference_from_dense(x)
    assert got.indices.dtype == torch.int32 and torch.equal(got.indices, want_i)
    assert got.features.dtype == dtype
    assert torch.equal(got.features.view(torch.uint8), want_f.contiguous().view(torch.uint8))   # bits, NaN included
    assert got.spatial_shape == list(shape[1:-1]) and got.batch_size == shape[0]


@pytest.mark.gpu
def test_round_trip_and_gradient():
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(2)
    x = (torch.randn(2, 20, 24, 16, 32, generator=g) * (torch.rand(2, 20, 24, 16, 1, generator=g) < 0.1)).cuda()
    x.requires_grad_(True)
    t = sp.SparseConvTensor.from_dense(x)
    assert torch.equal(t.dense(channels_first=False), x.detach())
    w = torch.randn(t.features.shape, generator=g).cuda()
    (t.features * w).sum().backward()
    xr = x.detach().clone().requires_grad_(True)
    vals, _ = reference_from_dense(xr)
    (vals * w).sum().backward()
    assert torch.equal(x.grad, xr.grad)


@pytest.mark.gpu
def test_all_zero_and_full():
    import spconv_triton_b200.pytorch as sp

    z = sp.SparseConvTensor.from_dense(torch.zeros(2, 4, 4, 4, 3, device="cuda"))
    assert z.features.shape == (0, 3) and z.indices.shape == (0, 4)
    f = sp.SparseConvTensor.from_dense(torch.ones(2, 4, 4, 4, 3, device="cuda"))
    assert f.features.shape == (128, 3) and f.indices[-1].tolist() == [1, 3, 3, 3]


@pytest.mark.gpu
def test_frozen_case():
    import spconv_triton_b200.pytorch as sp

    path = Path(__file__).parent / "golden" / "ref_add.pt"
    case = next((c for c in torch.load(path, weights_only=False).get("from_dense", [])), None)
    if case is None:
        pytest.skip("no frozen from_dense case in the fixture")
    t = sp.SparseConvTensor.from_dense(case["dense"].cuda())
    assert torch.equal(t.indices.cpu(), case["indices"]) and torch.equal(t.features.cpu(), case["features"])
