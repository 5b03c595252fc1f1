"""The native pass over a chain of convolutions (one library call for a whole
inference SparseSequential) against the same modules run one by one: identical
bits in the output tensor and in every rulebook cache entry, the pending
input-side tables included; the cases it must leave to the modules; the arena
retry."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _net_and_scene(batch=2):
    import bench

    torch.manual_seed(0)
    net = bench.init_backbone(bench.build_backbone()).half().eval().to(DEV)
    idx, feats = bench.make_scenes(3, n_scenes=1, batch=batch)[0]
    return net, idx.to(DEV), feats.to(DEV), bench.GRID, batch


def _run(net, idx, feats, grid, batch, native):
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200 import constants

    old = constants.SPCONV_NATIVE_SEQUENCE
    constants.SPCONV_NATIVE_SEQUENCE = native
    try:
        with torch.no_grad():
            out = net(sp.SparseConvTensor(feats, idx, grid, batch))
        torch.cuda.synchronize()
    finally:
        constants.SPCONV_NATIVE_SEQUENCE = old
    return out


def test_same_bits_as_the_modules_one_by_one():
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.pytorch import sequence

    net, idx, feats, grid, batch = _net_and_scene()
    with torch.no_grad():
        assert sequence.forward(net, sp.SparseConvTensor(feats, idx, grid, batch)) is not None
    a = _run(net, idx, feats, grid, batch, True)
    b = _run(net, idx, feats, grid, batch, False)
    assert a.spatial_shape == b.spatial_shape and a.batch_size == b.batch_size
    assert torch.equal(a.indices, b.indices) and torch.equal(a.features, b.features)
    assert sorted(a.indice_dict) == sorted(b.indice_dict)
    # the pass writes the column-major table only where one of its layers reads it (the 4 -> 16
    # stem runs on the CUDA cores); elsewhere it is made from the row-major copy when first read
    pending = [key for key, d in a.indice_dict.items() if d.__dict__.get("_pair_fwd_thunk") is not None]
    assert pending and len(pending) < len(a.indice_dict), pending
    # the pass orders the rows of a rulebook for its own GEMM tiles; the sorted masks and their
    # argsort, as the rulebook generator emits them, are made when read (and compared below)
    assert all(d.__dict__.get("_masks_fwd_thunk") is not None for d in a.indice_dict.values())
    for key in a.indice_dict:
        da, db = a.indice_dict[key], b.indice_dict[key]
        assert da.is_subm == db.is_subm and da.ksize == db.ksize and da.stride == db.stride
        assert da.spatial_shape == db.spatial_shape and da.out_spatial_shape == db.out_spatial_shape
        assert (da.out_indices is da.indices) == (db.out_indices is db.indices)  # subm: the same object
        for name in ("out_indices", "indices", "pair_fwd"):
            assert torch.equal(getattr(da, name), getattr(db, name)), (key, name)
        assert torch.equal(da.pair_fwd._spc_rowmajor, db.pair_fwd._spc_rowmajor)
        assert len(da.pair_mask_fwd_splits) == len(db.pair_mask_fwd_splits) == 1
        assert da.pair_mask_fwd_splits[0].shape == db.pair_mask_fwd_splits[0].shape
        assert torch.equal(da.pair_mask_fwd_splits[0], db.pair_mask_fwd_splits[0])
        assert torch.equal(da.mask_argsort_fwd_splits[0], db.mask_argsort_fwd_splits[0])
        assert np.array_equal(np.concatenate(da.masks), np.concatenate(db.masks))
        # the input-side tables: pending for strided layers, absent for submanifold ones in inference
        assert da.pair_bwd.shape == db.pair_bwd.shape and torch.equal(da.pair_bwd, db.pair_bwd), key
        assert len(da.pair_mask_bwd_splits) == len(db.pair_mask_bwd_splits)
        for ta, tb in zip(list(da.pair_mask_bwd_splits) + list(da.mask_argsort_bwd_splits),
                          list(db.pair_mask_bwd_splits) + list(db.mask_argsort_bwd_splits)):
            assert torch.equal(ta, tb)


def test_inverse_layer_reuses_a_rulebook_of_the_native_pass():
    import spconv_triton_b200.pytorch as sp

    net, idx, feats, grid, batch = _net_and_scene()
    torch.manual_seed(1)
    up = sp.SparseInverseConv3d(64, 32, 3, indice_key="down3", bias=False).half().eval().to(DEV)
    outs = []
    for native in (True, False):
        y = _run(net, idx, feats, grid, batch, native)
        with torch.no_grad():
            outs.append(up(y))
        torch.cuda.synchronize()
    assert torch.equal(outs[0].indices, outs[1].indices) and torch.equal(outs[0].features, outs[1].features)
    assert outs[0].spatial_shape == outs[1].spatial_shape


def test_cases_left_to_the_modules():
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.pytorch import sequence

    net, idx, feats, grid, batch = _net_and_scene()
    x = sp.SparseConvTensor(feats, idx, grid, batch)
    assert sequence.forward(net, x) is None  # autograd is on
    with torch.no_grad():
        assert sequence.forward(net, sp.SparseConvTensor(feats.float(), idx, grid, batch)) is None  # fp32 features
        net.train()
        assert sequence.forward(net, x) is None
        net.eval()
        assert sequence.forward(net, x) is not None
        mixed = sp.SparseSequential(sp.SubMConv3d(4, 16, 3, padding=1, indice_key="a"), sp.SparseMaxPool3d(2, 2))
        assert sequence.forward(mixed.half().eval().to(DEV), x) is None  # a pooling layer
        k5 = sp.SparseSequential(sp.SubMConv3d(4, 16, 5, padding=2))
        assert sequence.forward(k5.half().eval().to(DEV), x) is None  # Native algorithm (kv > 32)
        # a layer whose points vanish: the modules raise the reference's error
        gone = sp.SparseSequential(sp.SparseConv3d(4, 16, 1, stride=64, padding=0)).half().eval().to(DEV)
        far = idx.clone()
        far[:, 1:] = far[:, 1:] % 7 + 1
        with pytest.raises(ValueError, match="points vanished"):
            gone(sp.SparseConvTensor(feats, far, grid, batch))


def test_arena_that_is_too_small_is_retried():
    from spconv_triton_b200.pytorch import sequence

    net, idx, feats, grid, batch = _net_and_scene()
    expect = _run(net, idx, feats, grid, batch, False)
    old = sequence._ARENA_BYTES_PER_VOXEL, sequence._ARENA_MARGIN, sequence._ARENA_GRANULE
    sequence._ARENA_BYTES_PER_VOXEL, sequence._ARENA_MARGIN, sequence._ARENA_GRANULE = 64.0, 0, 4096
    net.__dict__.pop("_spc_plans", None)
    net.__dict__.pop("_spc_arena_floor", None)
    try:
        got = _run(net, idx, feats, grid, batch, True)
        assert next(iter(net.__dict__["_spc_plans"].values())).bytes_per_voxel > 64.0
    finally:
        sequence._ARENA_BYTES_PER_VOXEL, sequence._ARENA_MARGIN, sequence._ARENA_GRANULE = old
    assert torch.equal(got.indices, expect.indices) and torch.equal(got.features, expect.features)
    again = _run(net, idx, feats, grid, batch, True)  # sized from what the first pass needed
    assert torch.equal(again.features, expect.features)


def test_passes_in_flight_from_two_threads_give_the_same_results():
    """Independent passes issued by two worker threads, each on its own stream (their kernels overlap
    on the GPU), against the same passes one after the other."""
    import bench
    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.parallel import PassPipeline

    net, _, _, grid, batch = _net_and_scene()
    scenes = [(i.to(DEV), f.to(DEV)) for i, f in bench.make_scenes(5, n_scenes=3, batch=batch)]
    expect = [_run(net, i, f, grid, batch, True) for i, f in scenes]
    pipe = PassPipeline(torch.device(DEV, torch.cuda.current_device()), depth=2)
    futures = [pipe.submit(lambda i=i, f=f: net(sp.SparseConvTensor(f, i, grid, batch)))
               for _ in range(3) for i, f in scenes]
    got = [f.result() for f in futures]
    pipe.join()
    torch.cuda.synchronize()
    pipe.close()
    assert len(net.__dict__["_spc_plans"]) >= 2  # each thread compiled its own plan
    for k, g in enumerate(got):
        e = expect[k % len(scenes)]
        assert torch.equal(g.indices, e.indices) and torch.equal(g.features, e.features)
        for key in e.indice_dict:
            assert torch.equal(g.indice_dict[key].pair_fwd, e.indice_dict[key].pair_fwd)
            assert torch.equal(g.indice_dict[key].mask_argsort_fwd_splits[0], e.indice_dict[key].mask_argsort_fwd_splits[0])
