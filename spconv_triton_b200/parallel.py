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
    """Average the gradients of ``parameters`` over the default process group,
    blocking (one flat bucket).  ``GradientReducer`` is the overlapped form."""
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


class _Bucket:
    __slots__ = ("params", "views", "flat", "pending", "work", "ready")


class GradientReducer:
    """Data-parallel gradient averaging, bucketed and overlapped with backward.

    The reference leaves data parallelism to the user (its README tells users
    to wrap the model in DistributedDataParallel); this is the same exchange --
    one all-reduce (sum) of the parameter gradients per step, nothing else ever
    crosses GPUs -- arranged for sparse backbones, whose backward is a chain of
    short kernels: parameters are grouped into buckets in the order backward
    finishes them (last layer first); the moment the last gradient of a bucket
    has been accumulated, the bucket is flattened and its all-reduce is queued
    on a communication stream, so that NCCL runs beside the remaining input- and
    weight-gradient kernels.  ``finish()`` (after ``backward()``) makes the
    current stream wait for the buckets, divides by the world size and writes
    the averages back into ``p.grad``.

        reducer = GradientReducer(model.parameters())
        loss.backward()
        reducer.finish()
        optimizer.step()

    Works on CPU tensors with the gloo backend (no streams) for tests.
    """

    def __init__(self, parameters, bucket_bytes: int = 8 << 20, process_group=None):
        import torch.distributed as dist

        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        params = [p for p in parameters if p.requires_grad]
        self.buckets: list[_Bucket] = []
        self._bucket_of: dict = {}
        self._comm_stream = None
        self._handles = []
        self.launched_during_backward = 0
        cur, cur_bytes = [], 0
        for p in reversed(params):  # backward reaches the last layer's parameters first
            cur.append(p)
            cur_bytes += p.numel() * 4
            if cur_bytes >= bucket_bytes:
                self._add_bucket(cur)
                cur, cur_bytes = [], 0
        if cur:
            self._add_bucket(cur)
        for p in params:
            self._handles.append(p.register_post_accumulate_grad_hook(self._on_grad))

    def _add_bucket(self, params):
        b = _Bucket()
        b.params = list(params)
        dev = params[0].device
        b.flat = torch.zeros(sum(p.numel() for p in params), dtype=torch.float32, device=dev)
        b.views, off = [], 0
        for p in params:
            b.views.append(b.flat[off:off + p.numel()].view_as(p))
            off += p.numel()
        b.pending, b.work, b.ready = len(params), None, None
        for p in params:
            self._bucket_of[id(p)] = b
        self.buckets.append(b)

    def _stream(self, device):
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device, priority=-1)
        return self._comm_stream

    def _on_grad(self, p):
        b = self._bucket_of[id(p)]
        b.pending -= 1
        if b.pending == 0:
            self.launched_during_backward += 1
            self._launch(b)

    def _launch(self, b):
        import torch.distributed as dist

        grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in b.params]
        torch._foreach_copy_(b.views, grads)
        if self.world == 1:
            return
        if b.flat.is_cuda:
            comm = self._stream(b.flat.device)
            comm.wait_stream(torch.cuda.current_stream(b.flat.device))
            with torch.cuda.stream(comm):
                b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        else:
            b.work = dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def finish(self):
        """Call after ``backward()``: every bucket averaged and written back."""
        for b in self.buckets:
            if b.pending > 0:
                # parameters that took no part in this backward keep a zero (or their old) gradient
                if all(p.grad is None for p in b.params):
                    b.pending = len(b.params)
                    continue
                self._launch(b)
            if b.work is not None:
                if b.flat.is_cuda:
                    with torch.cuda.stream(self._stream(b.flat.device)):
                        b.work.wait()
                    torch.cuda.current_stream(b.flat.device).wait_stream(self._stream(b.flat.device))
                else:
                    b.work.wait()
                b.work = None
            if self.world > 1:
                b.flat.div_(self.world)
            targets = [p.grad for p in b.params if p.grad is not None]
            sources = [v for p, v in zip(b.params, b.views) if p.grad is not None]
            if targets:
                torch._foreach_copy_(targets, sources)
            b.pending = len(b.params)

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles.clear()


class PassPipeline:
    """Independent forward passes in flight from several host threads, one CUDA stream each.

    A pass over a sparse backbone blocks its host thread a few times (each strided layer reads its
    output count before it can size the next launch), so one thread cannot keep two passes in
    flight.  The library releases the interpreter lock while it waits, so ``depth`` worker threads,
    each issuing whole passes on its own stream, keep the GPU supplied with the kernels of ``depth``
    passes at once (throughput mode of an inference server; a single pass is not faster).

        pipe = PassPipeline(device, depth=2)
        futures = [pipe.submit(net, batch) for batch in batches]     # each returns net(batch)
        outputs = [f.result() for f in futures]
        pipe.join()                                                  # current stream waits for all passes
    """

    def __init__(self, device, depth: int = 2):
        import concurrent.futures
        import threading

        self.device = torch.device(device)
        self.depth = max(1, int(depth))
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=self.depth, thread_name_prefix="spc-pass")
        self._local = threading.local()
        self._streams: list = []
        self._lock = threading.Lock()
        self._origin = torch.cuda.current_stream(self.device)

    def _stream(self):
        st = getattr(self._local, "stream", None)
        if st is None:
            torch.cuda.set_device(self.device)
            st = torch.cuda.Stream(device=self.device)
            st.wait_stream(self._origin)  # set-up queued on the creating thread's stream comes first
            self._local.stream = st
            with self._lock:
                self._streams.append(st)
        return st

    def submit(self, fn, *args, **kwargs):
        """Runs ``fn(*args, **kwargs)`` on a worker thread under its stream (no autograd)."""

        def work():
            with torch.cuda.stream(self._stream()), torch.no_grad():
                return fn(*args, **kwargs)

        return self._pool.submit(work)

    def join(self):
        """Makes the current stream wait for everything the workers have issued so far
        (call it after the futures of interest have completed)."""
        cur = torch.cuda.current_stream(self.device)
        with self._lock:
            for st in self._streams:
                cur.wait_stream(st)

    def close(self):
        self._pool.shutdown(wait=True)


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
