"""The reference's frozen network-level golden cases, run on the GPU through
the public module API and the CUDA library (forward and backward)."""

import pytest
import torch

from frozen_cases import frozen, frozen_ids, run_net_case, run_pipeline_case

pytestmark = pytest.mark.gpu


@pytest.fixture
def sp():
    import spconv_triton_b200.pytorch as sp

    return sp


@pytest.mark.parametrize("case_id", frozen_ids("golden_ext_pool.pt"))
def test_pool_pipelines(sp, case_id):
    run_pipeline_case(sp, frozen("golden_ext_pool.pt", case_id), "cuda")


def test_seq2d_mixed(sp):
    run_pipeline_case(sp, frozen("golden_misc.pt", "seq2d_mixed"), "cuda")


@pytest.mark.parametrize("case_id", frozen_ids("golden_net.pt"))
def test_unet(sp, case_id):
    run_net_case(sp, frozen("golden_net.pt", case_id), "cuda")


def test_autocast_dtype_matrix(sp):
    """Under autocast a training forward returns fp16, an eval forward returns
    the weight dtype (the matrix the reference pins in
    tests/test_module_protocol.py:88-105)."""
    idx = torch.tensor([[0, 1, 1, 1], [0, 1, 1, 2], [0, 2, 2, 2], [0, 3, 1, 0]], dtype=torch.int32, device="cuda")
    feats = torch.randn(4, 16, device="cuda")
    layer = sp.SubMConv3d(16, 16, 3, indice_key="k").cuda()
    with torch.autocast("cuda", dtype=torch.float16):
        layer.train()
        assert layer(sp.SparseConvTensor(feats, idx, [4, 4, 4], 1)).features.dtype == torch.float16
        layer.eval()
        assert layer(sp.SparseConvTensor(feats, idx, [4, 4, 4], 1)).features.dtype == torch.float32


def test_folded_batchnorm_relu_matches_separate_modules(sp):
    """SparseSequential folds an inference [conv, BatchNorm1d, ReLU] into one
    kernel; the result must equal the three separate modules up to fp16 rounding
    of the intermediate, and the unfused path must still be selectable."""
    import numpy as np

    from gpu_util import unique_coords
    from spconv_triton_b200 import constants

    idx = torch.from_numpy(unique_coords(17, 20000, 2, [24, 64, 64])).cuda()
    torch.manual_seed(0)
    for dtype, tol in ((torch.float16, 3e-3), (torch.float32, 2e-5)):
        net = sp.SparseSequential(
            sp.SubMConv3d(16, 32, 3, padding=1, bias=False, indice_key="a"), torch.nn.BatchNorm1d(32), torch.nn.ReLU(),
            sp.SparseConv3d(32, 64, 3, stride=2, padding=1, bias=True), torch.nn.BatchNorm1d(64), torch.nn.ReLU(),
            sp.SubMConv3d(64, 64, 3, padding=1, bias=False, indice_key="b"), torch.nn.BatchNorm1d(64),
        ).cuda()
        with torch.no_grad():
            for m in net.modules():
                if isinstance(m, torch.nn.BatchNorm1d):
                    m.running_mean.normal_(0, 0.2)
                    m.running_var.uniform_(0.5, 1.5)
                    m.weight.uniform_(0.5, 1.5)
                    m.bias.normal_(0, 0.2)
        net = net.to(dtype).eval()
        feats = torch.randn(idx.shape[0], 16, device="cuda").to(dtype)
        outs = {}
        for fold in (True, False):
            constants.SPCONV_FOLD_BN_RELU = fold
            try:
                with torch.no_grad():
                    outs[fold] = net(sp.SparseConvTensor(feats, idx, [24, 64, 64], 2))
            finally:
                constants.SPCONV_FOLD_BN_RELU = True
        assert torch.equal(outs[True].indices, outs[False].indices)
        a, b = outs[True].features.double(), outs[False].features.double()
        assert (a - b).abs().max().item() <= tol * b.abs().max().item()
        # training mode never folds (BatchNorm uses batch statistics there)
        net.train()
        out_t = net(sp.SparseConvTensor(feats, idx, [24, 64, 64], 2))
        assert out_t.features.shape == outs[True].features.shape
