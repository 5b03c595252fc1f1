"""Network-level pins, no GPU: the reference's frozen golden cases (produced
upstream by CUDA spconv 2.3.8) run through this package's layers, autograd
functions and operator adaptors with the CPU oracle standing in for the CUDA
library.  Passing means (a) the oracle reproduces those goldens and (b) the
host-side logic (indice_key reuse, inverse-conv table swap, bias handling,
conv1x1 shortcut, canonical output order) matches the reference.
"""

import pytest
import torch

import oracle_backend
from frozen_cases import frozen, frozen_ids, run_net_case, run_pipeline_case


@pytest.fixture
def sp(monkeypatch):
    import spconv_triton_b200.pytorch as sp

    oracle_backend.install(monkeypatch)
    return sp


@pytest.mark.parametrize("case_id", frozen_ids("golden_ext_pool.pt"))
def test_pool_pipelines(sp, case_id):
    run_pipeline_case(sp, frozen("golden_ext_pool.pt", case_id), "cpu")


def test_seq2d_mixed(sp):
    run_pipeline_case(sp, frozen("golden_misc.pt", "seq2d_mixed"), "cpu")


@pytest.mark.parametrize("case_id", frozen_ids("golden_net.pt"))
def test_unet(sp, case_id):
    run_net_case(sp, frozen("golden_net.pt", case_id), "cpu")


def test_unet_state_dict_keys(sp):
    from frozen_cases import build_unet3d

    case = frozen("golden_net.pt", "unet3d_float32")
    assert sorted(build_unet3d(sp).state_dict().keys()) == sorted(case["state_dict"].keys())
