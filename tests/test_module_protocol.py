"""Drop-in protocol of the layer classes, against the reference's frozen
`golden_proto.pt` cases: seeded initialisation bit for bit, state_dict keys and
shapes, extra_repr, pickling, checkpoint hooks, constructor signatures."""

import inspect
import pickle

import pytest
import torch

from frozen_cases import frozen, frozen_ids

import spconv_triton_b200.pytorch as sp


def _cases(kind):
    return [i for i in frozen_ids("golden_proto.pt") if frozen("golden_proto.pt", i)["kind"] == kind]


@pytest.mark.parametrize("case_id", _cases("init"))
def test_seeded_init_bitwise(case_id):
    case = frozen("golden_proto.pt", case_id)
    torch.manual_seed(case["seed"])
    layer = getattr(sp, case["cls"])(**case["ctor"])
    assert list(layer.weight.shape) == case["expect"]["weight_shape"]
    assert torch.equal(layer.weight.detach(), case["expect"]["weight"])
    if case["expect"]["bias"] is None:
        assert layer.bias is None
    else:
        assert torch.equal(layer.bias.detach(), case["expect"]["bias"])


@pytest.mark.parametrize("case_id", _cases("state_dict_keys"))
def test_state_dict_keys(case_id):
    case = frozen("golden_proto.pt", case_id)
    sd = getattr(sp, case["cls"])(**case["ctor"]).state_dict()
    assert sorted(sd.keys()) == case["expect"]["keys"]
    for k, shape in case["expect"]["shapes"].items():
        assert list(sd[k].shape) == shape


@pytest.mark.parametrize("case_id", _cases("repr"))
def test_extra_repr(case_id):
    case = frozen("golden_proto.pt", case_id)
    assert getattr(sp, case["cls"])(**case["ctor"]).extra_repr() == case["expect"]["extra_repr"]


def test_pickle_roundtrip():
    layer = sp.SubMConv3d(4, 8, 3)
    assert torch.equal(layer.weight, pickle.loads(pickle.dumps(layer)).weight)
    x = sp.SparseConvTensor(torch.randn(5, 3), torch.zeros(5, 4, dtype=torch.int32), [4, 4, 4], 1)
    y = pickle.loads(pickle.dumps(x))
    assert torch.equal(x.features, y.features) and y.spatial_shape == [4, 4, 4]


def test_record_voxel_count_checkpoint_injection():
    sd = sp.SparseConv3d(4, 8, 3).state_dict()
    rvc = sp.SparseConv3d(4, 8, 3, record_voxel_count=True)
    missing, unexpected = rvc.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
    assert "max_num_voxels_during_training" in [n for n, _ in rvc.named_buffers()]
    assert sp.SparseConv3d(4, 8, 3).get_max_num_voxels() is None


CTOR = {
    "conv": ["in_channels", "out_channels", "kernel_size", "stride", "padding", "dilation", "groups", "bias",
             "indice_key", "algo", "fp32_accum", "record_voxel_count", "large_kernel_fast_algo", "name"],
    "inverse": ["in_channels", "out_channels", "kernel_size", "indice_key", "bias", "algo", "fp32_accum",
                "large_kernel_fast_algo", "name"],
    "subm": ["in_channels", "out_channels", "kernel_size", "stride", "padding", "dilation", "groups", "bias",
             "indice_key", "algo", "fp32_accum", "large_kernel_fast_algo", "name"],
    "pool": ["kernel_size", "stride", "padding", "dilation", "indice_key", "algo", "record_voxel_count", "name"],
}


def test_constructor_signatures():
    """Parameter names and order of the public layer classes (the reference pins
    them in tests/data/golden_api.json)."""
    def names(cls):
        return [p for p in inspect.signature(cls.__init__).parameters if p != "self"]

    for d in (1, 2, 3, 4):
        assert names(getattr(sp, f"SparseConv{d}d")) == CTOR["conv"]
        assert names(getattr(sp, f"SparseConvTranspose{d}d")) == CTOR["conv"]
        assert names(getattr(sp, f"SparseInverseConv{d}d")) == CTOR["inverse"]
        assert names(getattr(sp, f"SubMConv{d}d")) == CTOR["subm"]
        assert names(getattr(sp, f"SparseMaxPool{d}d")) == CTOR["pool"]
    for d in (1, 2, 3):
        assert names(getattr(sp, f"SparseAvgPool{d}d")) == CTOR["pool"]


def test_edge_behaviour_of_constructors_and_tensor():
    from spconv_triton_b200.core import ConvAlgo

    with pytest.raises(AssertionError):
        sp.SparseConv3d(4, 8, 3, groups=2)
    assert sp.SubMConv3d(4, 8, 5).algo == ConvAlgo.Native  # kv = 125 > 32
    assert sp.SubMConv3d(4, 8, 5, large_kernel_fast_algo=True).algo == ConvAlgo.MaskImplicitGemm
    assert sp.SparseConv3d(4, 8, 1).conv1x1 and not sp.SparseConv3d(4, 8, 1, stride=2).conv1x1
    with pytest.raises(AssertionError):
        sp.SparseAvgPool3d([4, 4, 4])  # kv = 64 > 32
    assert sp.SparseMaxPool3d(2).stride == [2, 2, 2]  # stride=None -> kernel size
    with pytest.raises(AssertionError, match="int32"):
        sp.SparseConvTensor(torch.randn(2, 3), torch.zeros(2, 4, dtype=torch.int64), [4, 4, 4], 1)
    x = sp.SparseConvTensor(torch.randn(2, 3), torch.zeros(2, 4, dtype=torch.int32), [4, 4, 4], 1)
    with pytest.raises(ValueError):
        x.features = torch.zeros(2, 3)
    y = x.replace_feature(x.features * 2)
    assert y.indice_dict is x.indice_dict and y.indices is x.indices


def test_runahead_plan_walk():
    """The rulebook run-ahead plans the sparse convolutions of nested
    SparseSequential containers in execution order and stops at the first
    sparse module whose output indices it cannot predict."""
    from torch import nn

    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.pytorch import runahead

    a, b, c, d = sp.SubMConv3d(4, 8, 3), sp.SparseConv3d(8, 8, 3, 2), sp.SubMConv3d(8, 8, 3), sp.SubMConv3d(8, 8, 3)
    net = sp.SparseSequential(a, nn.ReLU(), sp.SparseSequential(b, nn.BatchNorm1d(8), sp.SparseSequential(c)),
                              sp.SparseMaxPool3d(2, 2), d)
    assert runahead.flatten_convs(net) == [a, b, c]
    assert runahead.flatten_convs(sp.SparseSequential(nn.ReLU())) == []
    # CPU tensors never get a planner
    import torch

    x = sp.SparseConvTensor(torch.zeros(1, 4), torch.zeros(1, 4, dtype=torch.int32), [4, 4, 4], 1)
    assert runahead.begin(net, x) is None and x._planner is None


def test_posted_device_status_raises_at_the_next_pass():
    """A failure recorded by a kernel (a bounded wait that expired, an index row
    outside the grid) reaches the host through a mailbox word that the next
    forward pass looks at; here the word is set on the host side of the wrapper."""
    import pytest

    from spconv_triton_b200 import _lib

    _, view = _lib.status_mailbox(0)
    _lib.raise_posted_status()  # nothing posted: no error
    view[0] = _lib.SPC_ERR_DEVICE_WAIT_EXPIRED
    with pytest.raises(_lib.SpconvB200Error, match="bounded device-side wait") as e:
        _lib.raise_posted_status()
    assert e.value.status == _lib.SPC_ERR_DEVICE_WAIT_EXPIRED
    assert view[0] == 0  # delivered once
    _lib.raise_posted_status()
    view[0] = _lib.SPC_ERR_INVALID_ARGUMENT
    with pytest.raises(_lib.SpconvB200Error, match="outside batch_size"):
        _lib.raise_posted_status()


def test_native_sequence_plan():
    """Which containers the one-call inference pass takes, and how it maps layers to rulebooks
    (host logic only: the plan is compiled without touching the GPU)."""
    import bench
    from spconv_triton_b200.pytorch import sequence

    net = bench.build_backbone().eval()
    x = sp.SparseConvTensor(torch.zeros(5, 4), torch.zeros(5, 4, dtype=torch.int32), bench.GRID, 8)
    plan = sequence._compile(net, x)
    assert plan is not None and len(plan.steps) == len(bench.LAYERS)
    # layers that share an indice_key share the rulebook of the first of them
    assert [st.rulebook for st in plan.steps] == [0, 1, 2, 2, 4, 5, 5, 7, 8, 8]
    assert [st.generates for st in plan.steps] == [True, True, True, False, True, True, False, True, True, False]
    assert all(st.bn is not None and st.relu for st in plan.steps)
    assert plan.out_shape == [6, 200, 176]
    assert plan.layers[1].geom.subm == 0 and plan.layers[2].geom.subm == 1 and plan.layers[3].rulebook == 2
    # left to the modules: training mode, a pooling layer, a Native-algorithm layer, an inverse layer,
    # a rulebook that exists already
    assert sequence._compile(net.train(), x) is None
    net.eval()
    assert sequence._compile(sp.SparseSequential(sp.SubMConv3d(4, 8, 3, indice_key="a"), sp.SparseMaxPool3d(2, 2)).eval(), x) is None
    assert sequence._compile(sp.SparseSequential(sp.SubMConv3d(4, 8, 5)).eval(), x) is None
    assert sequence._compile(sp.SparseSequential(sp.SparseConv3d(4, 8, 3, 2, indice_key="d"),
                                                 sp.SparseInverseConv3d(8, 4, 3, indice_key="d")).eval(), x) is None
    x.indice_dict["subm0"] = object()
    assert sequence._compile(net, x) is None


def test_pending_column_major_table_of_a_cache_entry():
    """An indice_dict entry whose column-major pair table was not written hands out the transpose
    of the row-major copy at the first read, once, and an assignment replaces it."""
    from spconv_triton_b200.core import ConvAlgo
    from spconv_triton_b200.pytorch.core import ImplicitGemmIndiceData
    from spconv_triton_b200.pytorch.sequence import _column_major

    kv, n = 27, 5
    rowmajor = torch.arange(n * 28, dtype=torch.int32).reshape(n, 28)
    idx = torch.zeros((n, 4), dtype=torch.int32)
    data = ImplicitGemmIndiceData(idx, idx, None, torch.Tensor(), [], [], [], [], [], [4, 4, 4], [4, 4, 4], True,
                                  ConvAlgo.MaskImplicitGemm, [3] * 3, [1] * 3, [1] * 3, [1] * 3)
    calls = []

    def thunk():
        calls.append(1)
        return _column_major(rowmajor, kv, None)

    data._pair_fwd_thunk = thunk
    table = data.pair_fwd
    assert table.shape == (kv, n) and table.is_contiguous()
    assert torch.equal(table, rowmajor[:, :kv].t()) and table._spc_rowmajor is rowmajor
    assert data.pair_fwd is table and len(calls) == 1
    data.pair_fwd = rowmajor
    assert data.pair_fwd is rowmajor and len(calls) == 1


def test_pending_sorted_masks_of_a_cache_entry():
    """The sorted mask words and their argsort are made from the row-major table at the first read
    of either: ascending as unsigned, ties in row order."""
    from spconv_triton_b200.core import ConvAlgo
    from spconv_triton_b200.pytorch.core import ImplicitGemmIndiceData
    from spconv_triton_b200.pytorch.sequence import _exact_masks
    import functools

    kv = 27
    present = torch.tensor([[1, 0, 1], [0, 0, 1], [1, 0, 1], [0, 0, 0], [1, 1, 1]], dtype=torch.bool)
    rowmajor = torch.full((5, 28), -1, dtype=torch.int32)
    rowmajor[:, [0, 13, 26]] = torch.where(present, torch.arange(15, dtype=torch.int32).reshape(5, 3), -1)
    words = [(1 << 0) * int(p[0]) + (1 << 13) * int(p[1]) + (1 << 26) * int(p[2]) for p in present]
    idx = torch.zeros((5, 4), dtype=torch.int32)
    data = ImplicitGemmIndiceData(idx, idx, None, torch.Tensor(), None, [], None, [], [], [4, 4, 4], [4, 4, 4], True,
                                  ConvAlgo.MaskImplicitGemm, [3] * 3, [1] * 3, [1] * 3, [1] * 3)
    data._masks_fwd_thunk = functools.partial(_exact_masks, rowmajor, kv)
    order = sorted(range(5), key=lambda r: (words[r], r))
    assert data.mask_argsort_fwd_splits[0].tolist() == order
    assert data.pair_mask_fwd_splits[0][:, 0].tolist() == [words[r] for r in order]
    assert data.__dict__["_masks_fwd_thunk"] is None
