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
