"""World-size-2 checks of the multi-GPU host logic on CPU (gloo): sharding by
sample, independence of per-sample rulebooks, additive weight gradients,
gradient all-reduce and the throughput aggregation bench.py uses."""

import os
import socket
import sys
from pathlib import Path

import numpy as np
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist

    from gpu_util import unique_coords
    from oracle import features as of
    from oracle import rulebook as orb
    from spconv_triton_b200.parallel import GradientReducer, aggregate_throughput, allreduce_gradients, shard_by_sample

    dist.init_process_group("gloo", rank=rank, world_size=world)
    shape, batch, n = [12, 16, 14], 4, 1200
    idx = torch.from_numpy(unique_coords(9, n, batch, shape))
    g = torch.Generator().manual_seed(1)
    feats = torch.randn(n, 8, generator=g)
    w = torch.randn(6, 27, 8, generator=g) * 0.1
    gout_full = torch.randn(n, 6, generator=g)

    li, lf, lb = shard_by_sample(idx, feats, batch, rank, world)
    assert lb == 2 and int(li[:, 0].max()) == 1
    args = ([3] * 3, [1] * 3, [1] * 3, [1] * 3, [0] * 3, True, False, True, False)
    local = orb.igemm_pairs(li.numpy(), lb, shape, *args)
    out_local = of.conv_forward(lf, w, local[2], li.shape[0])

    # the same rows computed inside the full batch
    full = orb.igemm_pairs(idx.numpy(), batch, shape, *args)
    out_full = of.conv_forward(feats, w, full[2], n)
    keep = (idx[:, 0] % world) == rank
    assert torch.allclose(out_local, out_full[keep], atol=1e-6)

    # weight gradient: local contributions add up to the full-batch gradient
    dw_local = of.conv_backward_weight(lf, gout_full[keep], local[2], (6, 27, 8))
    p = torch.nn.Parameter(torch.zeros(6, 27, 8))
    p.grad = dw_local.clone()
    allreduce_gradients([p], world)
    dw_full = of.conv_backward_weight(feats, gout_full, full[2], (6, 27, 8))
    assert torch.allclose(p.grad * world, dw_full, atol=1e-5)

    # bucketed reducer: hooks fire during backward, finish() leaves the average in p.grad
    torch.manual_seed(3)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    reducer = GradientReducer(net.parameters(), bucket_bytes=256)
    assert len(reducer.buckets) >= 2
    for step in range(2):  # twice: the buckets re-arm
        net.zero_grad()
        x = torch.randn(5, 8, generator=torch.Generator().manual_seed(10 * step + rank))
        net(x).pow(2).sum().backward()
        reducer.finish()
        assert reducer.launched_during_backward == len(reducer.buckets) * (step + 1)
        expect = [torch.zeros_like(q) for q in net.parameters()]
        for r in range(world):
            ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
            ref.load_state_dict(net.state_dict())
            xr = torch.randn(5, 8, generator=torch.Generator().manual_seed(10 * step + r))
            ref(xr).pow(2).sum().backward()
            for e, q in zip(expect, ref.parameters()):
                e += q.grad / world
        for e, q in zip(expect, net.parameters()):
            assert torch.allclose(q.grad, e, atol=1e-5), (q.grad - e).abs().max()
    reducer.remove()

    units, ms = aggregate_throughput(float(li.shape[0]), 10.0 + rank)
    assert units == n and ms == 11.0
    dist.barrier()
    dist.destroy_process_group()
    Path(out_dir, f"ok{rank}").write_text("ok")


def test_two_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_shard_rebases_batch_column():
    sys.path.insert(0, str(ROOT))
    from spconv_triton_b200.parallel import shard_by_sample

    idx = torch.tensor([[0, 1], [1, 2], [2, 3], [3, 4], [4, 5]], dtype=torch.int32)
    feats = torch.arange(5.0).unsqueeze(1)
    li, lf, lb = shard_by_sample(idx, feats, 5, 1, 2)
    assert li.tolist() == [[0, 2], [1, 4]] and lf.squeeze(1).tolist() == [1.0, 3.0] and lb == 2
