"""SparseConvTensor.dense() on the GPU (one zero fill + one scatter kernel) against
the reference's definition, scatter_nd into zeros followed by permute + contiguous
(spconv_triton/pytorch/core.py:167-178,320-334), forward and gradient, bit for bit."""

import pytest
import torch

from gpu_util import DEV, unique_coords

pytestmark = pytest.mark.gpu


def reference_dense(features, indices, batch_size, spatial_shape, channels_first):
    shape = [batch_size, *spatial_shape, features.shape[1]]
    res = torch.zeros(shape, dtype=features.dtype, device=features.device)
    idx = indices.long()
    res[tuple(idx[:, i] for i in range(idx.shape[1]))] = features
    if not channels_first:
        return res
    nd = len(spatial_shape)
    return res.permute(0, nd + 1, *range(1, nd + 1)).contiguous()


@pytest.mark.parametrize("shape,batch,n,channels,dtype", [
    ([5, 20, 24], 3, 1500, 64, torch.float16), ([5, 20, 24], 2, 900, 130, torch.float32),
    ([40, 36], 2, 700, 7, torch.float32), ([9], 4, 30, 16, torch.bfloat16), ([3, 4, 5, 6], 2, 200, 33, torch.float64),
    ([8, 8, 8], 1, 1, 300, torch.float16)])
@pytest.mark.parametrize("channels_first", [True, False])
def test_dense_matches_definition(shape, batch, n, channels, dtype, channels_first):
    import spconv_triton_b200.pytorch as sp

    idx = torch.from_numpy(unique_coords(4, n, batch, shape)).to(DEV)
    feats = torch.randn(n, channels, generator=torch.Generator().manual_seed(1)).to(dtype).to(DEV).requires_grad_(True)
    x = sp.SparseConvTensor(feats, idx, shape, batch)
    out = x.dense(channels_first=channels_first)
    feats2 = feats.detach().clone().requires_grad_(True)
    exp = reference_dense(feats2, idx, batch, shape, channels_first)
    assert out.shape == exp.shape and out.dtype == exp.dtype
    assert torch.equal(out, exp)
    g = torch.randn(exp.shape, generator=torch.Generator().manual_seed(2)).to(dtype).to(DEV)
    out.backward(g)
    exp.backward(g)
    assert torch.equal(feats.grad, feats2.grad)


def test_dense_after_backbone_layer():
    """dense() of a layer's output (rows in the order the rulebook emits them)."""
    import spconv_triton_b200.pytorch as sp

    shape, batch = [12, 40, 44], 2
    idx = torch.from_numpy(unique_coords(8, 4000, batch, shape)).to(DEV)
    feats = torch.randn(4000, 16, device=DEV).half()
    net = sp.SparseSequential(sp.SparseConv3d(16, 32, 3, 2, 1), torch.nn.ReLU()).to(DEV).half().eval()
    with torch.no_grad():
        y = net(sp.SparseConvTensor(feats, idx, shape, batch))
    assert torch.equal(y.dense(), reference_dense(y.features, y.indices, batch, y.spatial_shape, True))
