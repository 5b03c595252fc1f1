"""One process, two GPUs: per-device state of the library (the dynamic shared memory opt-in of
the tcgen05 kernels, the status word, the scratch of the allocation-free weight gradient, the
multiprocessor count that sizes the weight-gradient split) must follow the current device.
Skipped on a single-GPU box."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_same_layers_on_two_devices_in_one_process():
    import spconv_triton_b200.pytorch as sp
    from gpu_util import unique_coords
    from spconv_triton_b200.pytorch._impl import gemm as G

    shape, batch, n = [24, 40, 36], 2, 9000
    idx = torch.from_numpy(unique_coords(3, n, batch, shape))
    torch.manual_seed(0)
    feats = torch.randn(n, 64).half()
    net = sp.SparseSequential(
        sp.SubMConv3d(64, 64, 3, padding=1, bias=False, indice_key="a"), torch.nn.BatchNorm1d(64), torch.nn.ReLU(),
        sp.SparseConv3d(64, 128, 3, stride=2, padding=1, bias=False, indice_key="d"), torch.nn.BatchNorm1d(128),
        torch.nn.ReLU()).half()
    results = []
    for dev in ("cuda:0", "cuda:1"):
        m = copy.deepcopy(net).to(dev)  # the training pass below moves the BatchNorm statistics
        # inference: the one-call pass (tcgen05 kernels with > 48 KB of shared memory)
        m.eval()
        with torch.no_grad():
            out = m(sp.SparseConvTensor(feats.to(dev), idx.to(dev), shape, batch))
        # training: forward, input and weight gradients through the modules
        m.train()
        x = feats.to(dev).requires_grad_(True)
        y = m(sp.SparseConvTensor(x, idx.to(dev), shape, batch))
        y.features.float().pow(2).sum().backward()
        torch.cuda.synchronize(dev)
        G.check_device_status(torch.device(dev))
        results.append((out.features.cpu(), out.indices.cpu(), x.grad.cpu(), m[0].weight.grad.cpu().clone()))
        m.zero_grad()
    a, b = results
    assert torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
    assert torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
