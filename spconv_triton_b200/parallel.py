"""Data parallelism by sample: the only way this path shards.

Rulebooks never pair voxels of different samples (the batch index is the most
significant digit of every linear coordinate), weights are replicated and the
weight gradient is additive over samples.  Inference therefore needs no
collective at all; training needs one all-reduce of the parameter gradients.
"""

from __future__ import annotations

import torch


def shard_by_sample(indices: torch.Tensor, features: torch.Tensor, batch_size: int, rank: int, world: int):
    """Rows of the samples ``b`` with ``b % world == rank``, with the batch
    column re-based to 0..local_batch-1.  Returns (indices, features, local_batch_size)."""
    b = indices[:, 0]
    keep = (b % world) == rank
    local = indices[keep].clone()
    local[:, 0] = torch.div(local[:, 0], world, rounding_mode="floor")
    n_local = len(range(rank, batch_size, world))
    return local, features[keep], n_local


def allreduce_gradients(parameters, world: int | None = None):
    """Sum-then-average the gradients of ``parameters`` over the default process
    group (one flat bucket; the parameter volume of sparse backbones is small)."""
    import torch.distributed as dist

    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return
    world = world or dist.get_world_size()
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    flat /= world
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g).to(g.dtype))
        off += n


def aggregate_throughput(local_units: float, local_ms: float, device=None):
    """(sum of units over ranks, max of milliseconds over ranks)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(local_units), float(local_ms)
    t = torch.tensor([local_units], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    m = torch.tensor([local_ms], dtype=torch.float64, device=device)
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    return float(t.item()), float(m.item())
