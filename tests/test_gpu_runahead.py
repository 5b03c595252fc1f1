"""Rulebook run-ahead of SparseSequential: building rulebooks on a second
stream must not change a single bit of any result, forward or backward, and
must fall back to the inline path wherever the look-ahead cannot predict."""

import numpy as np
import pytest
import torch
from torch import nn

from gpu_util import DEV, unique_coords

pytestmark = pytest.mark.gpu


@pytest.fixture
def sp():
    import spconv_triton_b200.pytorch as sp

    return sp


def _scene(seed, n, batch, shape, channels, dtype):
    idx = torch.from_numpy(unique_coords(seed, n, batch, shape)).to(DEV)
    gen = torch.Generator().manual_seed(seed)
    feats = torch.randn(n, channels, generator=gen).to(dtype).to(DEV)
    return idx, feats


def _unet(sp, c):
    """Encoder / decoder with shared subm keys, a stride-2 conv whose rulebook
    an inverse conv reuses, nested containers and dense modules in between."""
    return sp.SparseSequential(
        sp.SubMConv3d(c, 16, 3, indice_key="s1", bias=False), nn.BatchNorm1d(16), nn.ReLU(),
        sp.SparseSequential(sp.SubMConv3d(16, 16, 3, indice_key="s1"), nn.ReLU()),
        sp.SparseConv3d(16, 32, 3, stride=2, padding=1, indice_key="d1"), nn.BatchNorm1d(32), nn.ReLU(),
        sp.SubMConv3d(32, 32, 3, indice_key="s2"),
        sp.SparseConv3d(32, 32, [3, 1, 3], stride=[2, 1, 2], padding=[1, 0, 1], indice_key="d2"), nn.ReLU(),
        sp.SubMConv3d(32, 32, 3),
        sp.SparseInverseConv3d(32, 32, [3, 1, 3], indice_key="d2"),
        sp.SparseInverseConv3d(32, 16, 3, indice_key="d1"),
        sp.SubMConv3d(16, 16, 3, indice_key="s1"),
    )


def _run(sp, net, idx, feats, shape, batch, runahead, train):
    from spconv_triton_b200 import constants

    old = constants.SPCONV_RULEBOOK_RUNAHEAD
    constants.SPCONV_RULEBOOK_RUNAHEAD = runahead
    try:
        net.train(train)
        x_feats = feats.clone().requires_grad_(train)
        for p in net.parameters():
            p.grad = None
        with torch.set_grad_enabled(train):
            out = net(sp.SparseConvTensor(x_feats, idx, shape, batch))
            grads = None
            if train:
                out.features.float().square().sum().backward()
                grads = [x_feats.grad.clone()] + [p.grad.clone() for p in net.parameters()]
        torch.cuda.synchronize()
        assert out._planner is None
        return out, grads
    finally:
        constants.SPCONV_RULEBOOK_RUNAHEAD = old


@pytest.mark.parametrize("dtype,train", [(torch.float16, False), (torch.float32, False), (torch.float32, True)])
def test_identical_with_and_without(sp, dtype, train):
    shape, batch = [24, 40, 36], 3
    idx, feats = _scene(11, 30000, batch, shape, 8, dtype)
    torch.manual_seed(3)
    net = _unet(sp, 8).to(DEV).to(dtype)
    ref, ref_grads = _run(sp, net, idx, feats, shape, batch, False, train)
    for _ in range(3):  # repeated: stream hand-over and allocator reuse across forwards
        out, grads = _run(sp, net, idx, feats, shape, batch, True, train)
        assert torch.equal(out.indices, ref.indices)
        assert out.spatial_shape == ref.spatial_shape
        assert torch.equal(out.features, ref.features)
        assert set(out.indice_dict) == set(ref.indice_dict)
        for key, d in ref.indice_dict.items():
            e = out.indice_dict[key]
            assert torch.equal(e.pair_fwd, d.pair_fwd) and torch.equal(e.out_indices, d.out_indices)
            if d.pair_bwd is not None and d.pair_bwd.numel():
                assert torch.equal(e.pair_bwd, d.pair_bwd)
        if train:
            for a, b in zip(grads, ref_grads):
                assert torch.equal(a, b)


def test_planner_is_used(sp, monkeypatch):
    """The planned rulebooks are the ones consumed: every generating layer takes
    its rulebook from the planner, none is generated twice."""
    from spconv_triton_b200.pytorch import ops, runahead

    shape, batch = [24, 40, 36], 2
    idx, feats = _scene(5, 12000, batch, shape, 8, torch.float16)
    net = _unet(sp, 8).to(DEV).half().eval()
    calls, taken = [], []
    orig = ops.get_indice_pairs_implicit_gemm
    monkeypatch.setattr(ops, "get_indice_pairs_implicit_gemm", lambda *a, **k: calls.append(1) or orig(*a, **k))
    orig_take = runahead.RulebookPlanner.take

    def take(self, conv, x):
        res = orig_take(self, conv, x)
        taken.append(res is not None)
        return res

    monkeypatch.setattr(runahead.RulebookPlanner, "take", take)
    with torch.no_grad():
        net(sp.SparseConvTensor(feats, idx, shape, batch))
    # s1, d1, s2, d2 and the unnamed subm generate; reuse and inverse layers do not
    assert len(calls) == 5
    assert taken == [True] * 5


def test_errors_surface_at_the_layer(sp):
    """A rulebook that cannot be built while planning is not reported early: the
    layer itself raises, as it does without the run-ahead."""
    shape, batch = [8, 8, 8], 1
    idx = torch.tensor([[0, 1, 1, 1], [0, 2, 3, 1]], dtype=torch.int32, device=DEV)
    feats = torch.randn(2, 4, device=DEV)
    net = sp.SparseSequential(sp.SubMConv3d(4, 4, 3), sp.SubMConv3d(4, 4, [2, 2, 2]), sp.SubMConv3d(4, 4, 3)).to(DEV)
    with pytest.raises(NotImplementedError):  # even subm kernel sizes are rejected by the layer
        net(sp.SparseConvTensor(feats, idx, shape, batch))


def test_unknown_modules_end_the_plan(sp):
    """Pooling is not predicted: the plan stops there and the rest runs inline."""
    from spconv_triton_b200.pytorch import runahead

    net = sp.SparseSequential(sp.SubMConv3d(4, 8, 3), sp.SparseConv3d(8, 8, 3, 2), sp.SparseMaxPool3d(2, 2),
                              sp.SubMConv3d(8, 8, 3))
    assert len(runahead.flatten_convs(net)) == 2
    shape, batch = [16, 16, 16], 2
    idx, feats = _scene(2, 1500, batch, shape, 4, torch.float32)
    net = net.to(DEV)
    from spconv_triton_b200 import constants

    outs = []
    for flag in (False, True):
        old, constants.SPCONV_RULEBOOK_RUNAHEAD = constants.SPCONV_RULEBOOK_RUNAHEAD, flag
        try:
            with torch.no_grad():
                outs.append(net(sp.SparseConvTensor(feats, idx, shape, batch)))
        finally:
            constants.SPCONV_RULEBOOK_RUNAHEAD = old
    assert torch.equal(outs[0].features, outs[1].features) and torch.equal(outs[0].indices, outs[1].indices)


@pytest.mark.parametrize("runahead", [False, True])
def test_pending_input_side_tables(sp, runahead):
    """An inference forward of a strided layer leaves pair_bwd and its masks unbuilt;
    reading them from the indice_dict entry builds exactly what a training forward builds."""
    from spconv_triton_b200 import constants
    from spconv_triton_b200.pytorch._impl import pairs

    shape, batch = [20, 36, 32], 2
    idx, feats = _scene(21, 9000, batch, shape, 8, torch.float16)
    net = sp.SparseSequential(sp.SubMConv3d(8, 16, 3, indice_key="s"),
                              sp.SparseConv3d(16, 16, 3, stride=2, padding=1, indice_key="d")).to(DEV).half().eval()
    old, constants.SPCONV_RULEBOOK_RUNAHEAD = constants.SPCONV_RULEBOOK_RUNAHEAD, runahead
    try:
        with torch.no_grad():
            out = net(sp.SparseConvTensor(feats, idx, shape, batch))
    finally:
        constants.SPCONV_RULEBOOK_RUNAHEAD = old
    entry = out.indice_dict["d"]
    assert entry._late is not None  # nothing built yet
    full = pairs.igemm_pairs(idx, batch, shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, True, False)
    assert torch.equal(entry.pair_bwd, full[3])
    assert entry._late is None
    assert torch.equal(entry.pair_mask_bwd_splits[0], full[5][0])
    assert torch.equal(entry.mask_argsort_bwd_splits[0], full[7][0])
    assert torch.equal(entry.pair_fwd, full[2]) and torch.equal(entry.out_indices, full[0])
