"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[2], the configuration its metric is quoted on):
VoxelNet-style sparse middle encoder, fp16 inference: SubMConv3d 4->16, then
three stages of [SparseConv3d k3 s2 p1 + 2 x SubMConv3d k3] at 32 / 64 / 64
channels, BatchNorm + ReLU after every convolution, grid [41, 1600, 1408],
batch 8, 16k-24k voxels per sample drawn by the seeded plane-plus-clusters
generator (synthetic stand-in for LiDAR sweeps).  One step = one forward pass
over one batch; every step sees a different scene, so every step rebuilds its
seven rulebooks.  Metric: input Mvoxels/s.

With N > 1 (launched by torchrun, one rank per GPU) each rank runs its own
batches -- the path shards by sample and has no data-path collective -- and
the value is all ranks' voxels over the slowest rank's device time (weak
scaling).

``--impl reference`` times the CPU restatement of the reference's algorithm
(oracle/) on the host cores over a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GRID = [41, 1600, 1408]
BATCH = 8
N_RANGE = (16000, 24000)
N_SCENES = 4

# kind, c_in, c_out, kernel, stride, padding, indice_key
LAYERS = [
    dict(kind="subm", cin=4, cout=16, k=3, s=1, p=1, key="subm0"),
    dict(kind="conv", cin=16, cout=32, k=3, s=2, p=1, key="down1"),
    dict(kind="subm", cin=32, cout=32, k=3, s=1, p=1, key="subm1"),
    dict(kind="subm", cin=32, cout=32, k=3, s=1, p=1, key="subm1"),
    dict(kind="conv", cin=32, cout=64, k=3, s=2, p=1, key="down2"),
    dict(kind="subm", cin=64, cout=64, k=3, s=1, p=1, key="subm2"),
    dict(kind="subm", cin=64, cout=64, k=3, s=1, p=1, key="subm2"),
    dict(kind="conv", cin=64, cout=64, k=3, s=2, p=1, key="down3"),
    dict(kind="subm", cin=64, cout=64, k=3, s=1, p=1, key="subm3"),
    dict(kind="subm", cin=64, cout=64, k=3, s=1, p=1, key="subm3"),
]


def build_backbone():
    import spconv_triton_b200.pytorch as sp

    mods = []
    for L in LAYERS:
        if L["kind"] == "subm":
            mods.append(sp.SubMConv3d(L["cin"], L["cout"], L["k"], padding=L["p"], bias=False, indice_key=L["key"]))
        else:
            mods.append(sp.SparseConv3d(L["cin"], L["cout"], L["k"], stride=L["s"], padding=L["p"], bias=False,
                                        indice_key=L["key"]))
        mods.append(torch.nn.BatchNorm1d(L["cout"], eps=1e-3, momentum=0.01))
        mods.append(torch.nn.ReLU())
    return sp.SparseSequential(*mods)


def init_backbone(net, seed=0):
    """Random-init weights; BatchNorm gets non-trivial inference statistics."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for m in net.modules():
            if isinstance(m, torch.nn.BatchNorm1d):
                m.weight.copy_(1 + 0.1 * torch.randn(m.num_features, generator=g))
                m.bias.copy_(0.1 * torch.randn(m.num_features, generator=g))
                m.running_mean.copy_(0.1 * torch.randn(m.num_features, generator=g))
                m.running_var.copy_(0.5 + torch.rand(m.num_features, generator=g))
            elif hasattr(m, "weight_shape"):
                fan_in = int(np.prod(m.weight_shape[1:]))
                m.weight.copy_(torch.randn(m.weight_shape, generator=g) * (2.0 / fan_in) ** 0.5)
    return net


def oracle_params(net):
    """The same weights, as the plain dicts oracle.backbone.run_backbone takes."""
    mods = list(net._modules.values())
    params = []
    for i in range(0, len(mods), 3):
        conv, bn = mods[i], mods[i + 1]
        w = conv.weight.detach().float().cpu()
        params.append(dict(weight=w.reshape(w.shape[0], -1, w.shape[-1]), bn_weight=bn.weight.detach().float().cpu(),
                           bn_bias=bn.bias.detach().float().cpu(), bn_mean=bn.running_mean.detach().float().cpu(),
                           bn_var=bn.running_var.detach().float().cpu(), eps=bn.eps))
    return params


def make_scenes(rank, n_scenes=N_SCENES, batch=BATCH):
    from spconv_triton_b200.scenes import lidar_like_batch

    scenes = []
    for s in range(n_scenes):
        idx = lidar_like_batch(1000 * (rank + 1) + s, batch, N_RANGE, tuple(GRID))
        g = torch.Generator().manual_seed(77 + 1000 * rank + s)
        feats = torch.rand(idx.shape[0], 4, generator=g).half()
        scenes.append((torch.from_numpy(idx), feats))
    return scenes


UNET_GRID = [512, 512, 64]
UNET_BATCH = 8
UNET_N_RANGE = (100000, 200000)
UNET_WIDTHS = (32, 64, 128, 256)


def build_unet(c_in=4, widths=UNET_WIDTHS):
    """BASELINE configs[3]: encoder of SubM / stride-2 convolutions at 32 / 64 / 128 / 256
    channels, decoder of SparseInverseConv3d layers that reuse the encoder's
    indice_keys, BatchNorm + ReLU after every convolution."""
    import spconv_triton_b200.pytorch as sp

    def block(conv, c):
        return [conv, torch.nn.BatchNorm1d(c, eps=1e-3, momentum=0.01), torch.nn.ReLU()]

    mods = block(sp.SubMConv3d(c_in, widths[0], 3, padding=1, bias=False, indice_key="subm0"), widths[0])
    for lvl in range(1, len(widths)):
        mods += block(sp.SparseConv3d(widths[lvl - 1], widths[lvl], 3, stride=2, padding=1, bias=False,
                                      indice_key=f"down{lvl}"), widths[lvl])
        mods += block(sp.SubMConv3d(widths[lvl], widths[lvl], 3, padding=1, bias=False, indice_key=f"subm{lvl}"),
                      widths[lvl])
    for lvl in range(len(widths) - 1, 0, -1):
        mods += block(sp.SparseInverseConv3d(widths[lvl], widths[lvl - 1], 3, indice_key=f"down{lvl}", bias=False),
                      widths[lvl - 1])
        mods += block(sp.SubMConv3d(widths[lvl - 1], widths[lvl - 1], 3, padding=1, bias=False,
                                    indice_key=f"subm{lvl - 1}"), widths[lvl - 1])
    return sp.SparseSequential(*mods)


def make_unet_scenes(n_scenes=2, batch=UNET_BATCH, n_range=UNET_N_RANGE, grid=UNET_GRID):
    """Indoor-like surface scenes; the same on every rank (each rank then keeps its samples)."""
    from spconv_triton_b200.scenes import indoor_like_batch

    scenes = []
    for s in range(n_scenes):
        idx = indoor_like_batch(500 + s, batch, n_range, tuple(grid))
        g = torch.Generator().manual_seed(900 + s)
        scenes.append((torch.from_numpy(idx), torch.rand(idx.shape[0], 4, generator=g)))
    return scenes


def run_train_arm(dev, rank, world, steps, warmup):
    """BASELINE configs[3]: one training step = forward + backward of the sparse
    UNet under fp16 autocast, the data-parallel all-reduce of the parameter
    gradients (bucketed, overlapped with backward) and an SGD update.  The batch
    of 8 samples is sharded by sample over the ranks (strong scaling); returns
    the record rank 0 adds to the JSON line."""
    import torch.distributed as dist

    import spconv_triton_b200.pytorch as sp
    from spconv_triton_b200.parallel import GradientReducer, shard_by_sample

    torch.manual_seed(1234)
    net = build_unet().to(dev).train()
    opt = torch.optim.SGD(net.parameters(), lr=1e-7, momentum=0.0)  # random targets: the step runs, the weights barely move
    n_params = sum(p.numel() for p in net.parameters())
    scenes, voxels = [], []
    for idx, feats in make_unet_scenes():
        li, lf, lb = shard_by_sample(idx, feats, UNET_BATCH, rank, world)
        scenes.append((li.to(dev), lf.to(dev), lb))
        voxels.append(int(idx.shape[0]))

    def step(i, reducer):
        idx, feats, lb = scenes[i % len(scenes)]
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.float16):
            out = net(sp.SparseConvTensor(feats, idx, UNET_GRID, lb))
            loss = out.features.float().pow(2).sum() / 1024.0  # keeps fp16 gradients in the normal range
        loss.backward()
        if reducer is not None:
            reducer.finish()
        opt.step()
        return loss

    mallocs = []  # device allocations inside each timed region

    def timed(reducer):
        for i in range(warmup):
            step(i, reducer)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        mallocs0 = torch.cuda.memory_stats(dev).get("num_device_alloc", 0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            loss = step(i, reducer)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        mallocs.append(torch.cuda.memory_stats(dev).get("num_device_alloc", 0) - mallocs0)
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, float(loss.detach())

    reducer = GradientReducer(net.parameters(), bucket_bytes=4 << 20) if world > 1 else None
    ms, loss = timed(reducer)
    rec = {
        "workload": "BASELINE configs[3]: sparse UNet 32/64/128/256 with SparseInverseConv3d decoder, fp16 autocast, "
                    "forward + backward + gradient all-reduce + SGD step, grid [512,512,64], batch 8 over all ranks",
        "scaling": "strong", "n_gpus": world, "steps": steps, "warmup": warmup,
        "voxels_per_step": int(np.mean(voxels)), "ms_per_step": ms / steps,
        "mvoxels_per_s": sum(voxels[i % len(voxels)] for i in range(steps)) / (ms * 1e-3) / 1e6,
        "parameters": n_params, "loss": loss, "device_mallocs_in_timed_region": mallocs[0],
    }
    if reducer is not None:
        # the same steps without the exchange: the difference is what the all-reduce costs when overlapped
        reducer.remove()
        ms_local, _ = timed(None)
        rec["allreduce"] = {"backend": "nccl", "buckets": len(reducer.buckets), "bytes_per_step": 4 * n_params,
                            "launched_during_backward": bool(reducer.launched_during_backward),
                            "ms_per_step_without": ms_local / steps,
                            "exposed_ms_per_step": (ms - ms_local) / steps}
    return rec


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, sampled every 100 ms by
    an ``nvidia-smi`` child process (a separate process, so that the queries do
    not contend with this process's CUDA calls).  ``window()`` marks the part of
    the log that belongs to the timed regions."""

    _FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
               "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
               "clocks_event_reasons.sw_power_cap")
    _NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        import shutil
        import subprocess
        import tempfile

        self._proc = None
        self._t0 = self._t1 = None
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        self._log = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self._proc = subprocess.Popen([exe, "-i", str(index), f"--query-gpu={self._FIELDS}",
                                           "--format=csv,noheader,nounits", "-lms", "100"],
                                          stdout=self._log, stderr=subprocess.DEVNULL)
        except Exception:
            self._proc = None

    def open_window(self):
        self._t0 = time.time()

    def close_window(self):
        self._t1 = time.time()

    def stop(self):
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()

    def summary(self):
        import datetime

        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self._proc is None:
            return out
        self.stop()
        self._log.flush()
        rows = []
        for line in open(self._log.name):
            parts = [x.strip() for x in line.split(",")]
            if len(parts) != 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), parts[4:]))
            except ValueError:
                continue
        os.unlink(self._log.name)
        if not rows:
            return out
        inside = [r for r in rows if self._t0 is not None and self._t0 - 0.1 <= r[0] <= self._t1 + 0.1] or rows[-3:]
        out["sm_mhz"] = statistics.median(r[1] for r in inside)
        out["sm_max_mhz"] = inside[0][2]
        out["samples"] = len(inside)
        out["reasons"] = sorted({n for r in inside for n, v in zip(self._NAMES, r[3]) if v.lower().startswith("active")})
        return out


def captured_gemm_traffic():
    """DRAM bytes (read + write) per forward gather-GEMM launch of this workload,
    from the committed summary of an ncu capture of this file, or None."""
    f = ROOT / "profiles" / "gather_gemm_backbone_dram_traffic.txt"
    if not f.exists():
        return None, None
    vals = {}
    for line in f.read_text().splitlines():
        if ":" in line and not line.lstrip().startswith("#"):
            k, v = line.split(":", 1)
            vals[k.strip()] = v.strip()
    try:
        return float(vals["dram_bytes_per_launch"]), vals.get("source")
    except (KeyError, ValueError):
        return None, None


class GemmProfiler:
    """Wraps the forward gather-GEMM wrapper so that every launch inside the
    timed region is bracketed by CUDA events on the launching stream and its
    algorithmic bytes and FLOPs are recorded."""

    def __init__(self):
        from spconv_triton_b200.pytorch import ops

        self.ops = ops
        self.records = []
        self.enabled = False
        self.count_pairs = False
        self.pairs = {}
        self.scene = 0
        self.call = 0
        self._orig = ops._gemm.conv_forward

    def install(self):
        orig = self._orig

        def wrapped(features, w, pair_fwd, n_out, *a, **kw):
            if not self.enabled:
                return orig(features, w, pair_fwd, n_out, *a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(features, w, pair_fwd, n_out, *a, **kw)
            e1.record()
            if self.count_pairs:  # untimed warm-up pass: remember the pair count of this call slot
                self.pairs[(self.scene, self.call)] = int((pair_fwd >= 0).sum().item())
            self.records.append((e0, e1, self.scene, self.call, tuple(pair_fwd.shape), features.shape[1],
                                 w.shape[0], features.element_size(), out.element_size(), features.shape[0]))
            self.call += 1
            return out

        self.ops._gemm.conv_forward = wrapped

    def summarize(self):
        """Aggregate over all recorded launches: FLOPs = 2*pairs*C_in*C_out;
        gathered bytes = gathered rows (pairs*C_in*e) + stored rows
        (n_out*C_out*e) + table (kv*n_out*4) + weights (kv*C_in*C_out*e);
        compulsory bytes = the same with every input row counted once
        (n_in*C_in*e), i.e. what has to cross the HBM interface when the
        repeated gathers hit in L2."""
        tot_ms = tot_bytes = tot_flops = tot_compulsory = 0.0
        for e0, e1, scene, call, (kv, n_out), cin, cout, e_in, e_out, n_in in self.records:
            pairs = self.pairs[(scene, call)]
            tot_ms += e0.elapsed_time(e1)
            tot_bytes += pairs * cin * e_in + n_out * cout * e_out + kv * n_out * 4 + kv * cin * cout * e_in
            # every input row once, however many outputs gather it
            tot_compulsory += n_in * cin * e_in + n_out * cout * e_out + kv * n_out * 4 + kv * cin * cout * e_in
            tot_flops += 2.0 * pairs * cin * cout
        n = max(len(self.records), 1)
        per_layer = {}
        for e0, e1, scene, call, (kv, n_out), cin, cout, e_in, e_out, n_in in self.records:
            rec = per_layer.setdefault(call, dict(layer=call, channels=f"{cin}->{cout}", launches=0, ms=0.0, flops=0.0))
            rec["launches"] += 1
            rec["ms"] += e0.elapsed_time(e1)
            rec["flops"] += 2.0 * self.pairs[(scene, call)] * cin * cout
        layers = [dict(layer=r["layer"], channels=r["channels"], avg_ms=r["ms"] / r["launches"],
                       tflops=r["flops"] / (r["ms"] * 1e-3) / 1e12 if r["ms"] else 0.0)
                  for r in sorted(per_layer.values(), key=lambda r: r["layer"])]
        return dict(launches=len(self.records), ms=tot_ms, bytes=tot_bytes, flops=tot_flops,
                    compulsory=tot_compulsory, avg_ms=tot_ms / n, layers=layers)


class RulebookProfiler:
    """CUDA events around every rulebook generation (one per distinct indice_key
    and forward) on the stream it is issued on; used with the run-ahead off."""

    def __init__(self, keys):
        from spconv_triton_b200.pytorch import ops

        self.ops, self.keys = ops, keys
        self.enabled = False
        self.call = 0
        self.records = []
        self._orig = ops.get_indice_pairs_implicit_gemm

    def install(self):
        orig = self._orig

        def wrapped(*a, **kw):
            if not self.enabled:
                return orig(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            res = orig(*a, **kw)
            e1.record()
            self.records.append((self.keys[self.call % len(self.keys)], e0, e1))
            self.call += 1
            return res

        self.ops.get_indice_pairs_implicit_gemm = wrapped

    def summarize(self, steps):
        per_key = {}
        for key, e0, e1 in self.records:
            per_key[key] = per_key.get(key, 0.0) + e0.elapsed_time(e1)
        per_key = {k: v / steps for k, v in per_key.items()}
        return per_key, sum(per_key.values())


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs"), d.get("bf16_tflops"), "measured"
    return 6650.0, 1590.0, "fallback"


def run_reference_arm(args):
    """CPU restatement of the reference's algorithm on the host cores: each
    step is one sample (16k-24k voxels) of the workload through the whole
    backbone; Mvoxels/s over K such steps."""
    from oracle.backbone import run_backbone

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    net = init_backbone(build_backbone())
    params = oracle_params(net)
    scenes = make_scenes(0, n_scenes=max(1, min(args.steps + args.warmup, 4)), batch=1)
    times, voxels = [], []
    for i in range(args.warmup + args.steps):
        idx, feats = scenes[i % len(scenes)]
        t0 = time.perf_counter()
        run_backbone(LAYERS, params, idx.numpy(), feats.float(), GRID, 1, acc_dtype=torch.float32)
        dt = time.perf_counter() - t0
        if i >= args.warmup:
            times.append(dt)
            voxels.append(idx.shape[0])
    value = sum(voxels) / sum(times) / 1e6
    line = {
        "impl": "reference", "metric": "voxelnet_backbone_fwd_mvoxels_per_s", "value": value, "unit": "Mvoxels/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "BASELINE configs[2]: VoxelNet-style backbone, one sample per step (bounded sample)",
                   "grid": GRID, "voxels_per_sample": list(N_RANGE)},
        "cpu_baseline": {"value": value, "unit": "Mvoxels/s", "cores": cores, "kind": "port",
                         "sample": f"{args.steps} steps of one sample each ({int(np.mean(voxels))} voxels avg), "
                                   "numpy rulebook + torch CPU fp32 gather-matmul"},
        "e2e": {"value": value, "unit": "Mvoxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def import_reference_gpu():
    """The reference project's own package (its Triton kernels, JIT-compiled for
    this GPU) from the git-ignored copy under baseline/_ref/, or None.  The
    package reads its version from installed-distribution metadata, which a
    plain copy does not have, so that one lookup is answered here."""
    ref = ROOT / "baseline" / "_ref" / "reference"
    if not (ref / "spconv_triton" / "__init__.py").is_file():
        return None
    import importlib
    import importlib.metadata as md

    orig = md.version
    md.version = lambda name: "1.0.0" if name == "spconv-triton" else orig(name)
    if str(ref) not in sys.path:
        sys.path.insert(0, str(ref))
    try:
        return importlib.import_module("spconv_triton.pytorch")
    finally:
        md.version = orig


def published_shape_scene(seed=42, n=50000):
    """The shape the reference's README quotes its timings on: one sample of ~50k
    voxels in a [41, 1600, 1408] grid (plane + clusters generator)."""
    from spconv_triton_b200.scenes import lidar_like_batch

    return torch.from_numpy(lidar_like_batch(seed, 1, (n, n), tuple(GRID)))


def run_published(sp, tag, dev, iters, constants_mod):
    """One layer, forward only, C_in = C_out = 256, k = 3, batch 1, ~50k voxels:
    SubMConv3d with its rulebook cached, SparseConv3d s2 and SparseConvTranspose3d
    s2 with the rulebook rebuilt every pass; fp16, TF32 and fp32.  ``sp`` is the
    ``...pytorch`` module of the implementation under test (same API for both)."""
    idx = published_shape_scene().to(dev)
    n = int(idx.shape[0])

    def timed(fn):
        for _ in range(max(10, iters // 5)):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / iters)
        return statistics.median(ts)

    for prec in ("fp16", "tf32", "fp32"):
        dtype = torch.float16 if prec == "fp16" else torch.float32
        constants_mod.SPCONV_ALLOW_TF32 = prec == "tf32"
        torch.manual_seed(0)
        feats = torch.randn(n, 256, device=dev).to(dtype)
        layers = {
            "subm_cached": sp.SubMConv3d(256, 256, 3, padding=1, bias=False, indice_key="k"),
            "sparse_s2": sp.SparseConv3d(256, 256, 3, stride=2, padding=1, bias=False),
            "transpose_s2": sp.SparseConvTranspose3d(256, 256, 3, stride=2, padding=1, bias=False),
        }
        for name, layer in layers.items():
            layer = layer.to(dev).to(dtype).eval()
            x = sp.SparseConvTensor(feats, idx, GRID, 1)
            with torch.no_grad():
                out = layer(x)
                if name == "subm_cached":
                    x.indice_dict["k"] = out.indice_dict["k"]  # later passes reuse the rulebook
                ms = timed(lambda: layer(x))
            print(json.dumps({"op": f"published_{name}_{prec}", "impl": tag, "ms": ms, "voxels": n,
                              "n_out": int(out.features.shape[0]), "channels": 256}), flush=True)
    constants_mod.SPCONV_ALLOW_TF32 = False


def run_backbone_reference_gpu(dev, steps, warmup):
    """The reference's own modules and Triton kernels on this GPU over the
    headline workload (same network, weights, scenes and timing as the device-
    resident arm of the headline line)."""
    sp_ref = import_reference_gpu()
    if sp_ref is None:
        print(json.dumps({"op": "backbone_reference_gpu", "unavailable": "no copy of the reference under baseline/_ref"}))
        return
    ours = init_backbone(build_backbone())
    mods = []
    for L in LAYERS:
        if L["kind"] == "subm":
            mods.append(sp_ref.SubMConv3d(L["cin"], L["cout"], L["k"], padding=L["p"], bias=False, indice_key=L["key"]))
        else:
            mods.append(sp_ref.SparseConv3d(L["cin"], L["cout"], L["k"], stride=L["s"], padding=L["p"], bias=False,
                                            indice_key=L["key"]))
        mods.append(torch.nn.BatchNorm1d(L["cout"], eps=1e-3, momentum=0.01))
        mods.append(torch.nn.ReLU())
    net = sp_ref.SparseSequential(*mods)
    net.load_state_dict(ours.state_dict())
    net = net.half().eval().to(dev)
    scenes = [(i.to(dev), f.to(dev)) for i, f in make_scenes(0)]
    voxels = [int(i.shape[0]) for i, _ in scenes]

    def forward(s):
        idx, feats = scenes[s % len(scenes)]
        with torch.no_grad():
            return net(sp_ref.SparseConvTensor(feats, idx, GRID, BATCH))

    t0 = time.perf_counter()
    for w in range(max(warmup, 2 * len(scenes))):  # JIT compilation and autotuning happen here
        forward(w)
    torch.cuda.synchronize()
    warm_s = time.perf_counter() - t0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(steps):
        forward(s)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    total = sum(voxels[s % len(voxels)] for s in range(steps))
    print(json.dumps({"op": "backbone_reference_gpu", "impl": "reference (Triton kernels on this GPU)",
                      "metric": "voxelnet_backbone_fwd_mvoxels_per_s", "value": total / (ms * 1e-3) / 1e6,
                      "unit": "Mvoxels/s", "ms_per_step": ms / steps, "steps": steps,
                      "warmup_and_compile_s": warm_s}), flush=True)


def blob_scene(seed, batch, n_per_sample, grid=256):
    """Dense-ish random blobs (BASELINE configs[4]): n_per_sample unique voxels per sample filling
    random solid blobs of a grid^3 volume to 30 % occupancy."""
    from spconv_triton_b200.scenes import blob_batch

    return torch.from_numpy(blob_batch(seed, batch, n_per_sample, grid, 0.3))


def run_op_bench(args):
    """Single-operator timings at the other BASELINE configurations (not the
    headline line): ``--op pool`` = configs[4] SparseMaxPool3d k2 s2 and
    SparseAvgPool3d k3 s1 at C = 256 fp16, 4 x 400k voxels in 256^3;
    ``--op conv_s2`` = configs[1] SparseConv3d k3 s2 64 -> 128 fp16, 4 x 120k
    voxels; ``--op conv_subm`` = SubMConv3d k3 (forward, input and weight gradient)
    at 32, 64 and 128 channels on the voxel set two stride-2 layers leave of a
    4-sample LiDAR-like batch; ``--op voxelize`` = PointToVoxel on 1.2M points.
    One JSON line per kernel with algorithmic GB/s (and TFLOP/s)."""
    from spconv_triton_b200.pytorch._impl import gemm as G
    from spconv_triton_b200.pytorch._impl import pairs as P
    from spconv_triton_b200.pytorch._impl import pool as PL
    from spconv_triton_b200.scenes import lidar_like_batch

    dev = torch.device("cuda", 0)
    hbm_peak, tensor_peak, peak_kind = measured_peaks()

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def emit(name, ms, nbytes, flops=None, **extra):
        line = {"op": name, "ms": ms, "algorithmic_GBps": nbytes / ms / 1e6, "hbm_frac": nbytes / ms / 1e6 / hbm_peak,
                "peak_kind": peak_kind, **extra}
        if "gathered_bytes" in line:
            line["gathered_GBps"] = line.pop("gathered_bytes") / ms / 1e6
        if "mpoints_per_s" in line:
            line["mpoints_per_s"] = line["points"] / ms / 1e3
        if flops:
            line["TFLOPs"] = flops / ms / 1e9
            line["tensor_frac"] = flops / ms / 1e9 / tensor_peak
        print(json.dumps(line), flush=True)

    iters = max(args.steps, 5)
    if args.op == "published":
        import spconv_triton_b200.pytorch as sp
        from spconv_triton_b200 import constants

        run_published(sp, "spconv_triton_b200", dev, max(args.steps, 50), constants)
        return
    if args.op == "published_reference":
        sp_ref = import_reference_gpu()
        if sp_ref is None:
            print(json.dumps({"op": "published_reference", "unavailable": "no copy of the reference under baseline/_ref"}))
            return
        import spconv_triton.constants as ref_constants

        run_published(sp_ref, "reference (Triton kernels on this GPU)", dev, max(args.steps, 50), ref_constants)
        return
    if args.op == "backbone_reference_gpu":
        run_backbone_reference_gpu(dev, max(args.steps, 5), args.warmup)
        return
    if args.op == "conv_k5":
        # BASELINE configs[4]: SubMConv3d k5 256 -> 256 fp16 (kv 125, Native rulebook) on 4 x 400k blob voxels
        batch, c, n_per = 4, 256, args.k5_voxels
        idx = blob_scene(7, batch, n_per).to(dev)
        n = int(idx.shape[0])
        t0 = time.perf_counter()
        _, pair, npl = P.native_pairs(idx, batch, [256] * 3, [5] * 3, [1] * 3, [2] * 3, [1] * 3, [0] * 3, True, False)
        pf, pb = P.native_pair_to_tables(pair, npl, n, n, False)
        torch.cuda.synchronize()
        rb_ms = 1e3 * (time.perf_counter() - t0)
        del pair
        kv = int(pf.shape[0])
        pairs = int((pf >= 0).sum())
        x = torch.randn(n, c, device=dev).half()
        w = (torch.randn(c, kv, c, device=dev) * 0.01).half()
        g = torch.randn(n, c, device=dev).half()
        flops = 2.0 * pairs * c * c
        compulsory = 2 * n * c * 2 + kv * n * 4 + kv * c * c * 2
        it = max(3, min(iters, 10))
        emit("subm_k5_fwd_256_256", timed(lambda: G.conv_forward(x, w, pf, n), it), compulsory, flops, voxels=n,
             pairs=pairs, kv=kv, rulebook_first_call_ms=rb_ms)
        emit("subm_k5_dgrad_256_256", timed(lambda: G.conv_backward_input(g, w, pb, n), it), compulsory, flops)
        emit("subm_k5_wgrad_256_256", timed(lambda: G.conv_backward_weight(x, g, pf, (c, kv, c)), it),
             2 * n * c * 2 + kv * n * 4 + kv * c * c * 2, flops)
        return
    if args.op == "pool":
        batch, c = 4, 256
        idx = blob_scene(7, batch, args.pool_voxels)
        if args.voxel_order == "sorted":   # the order every rulebook of this library emits its outputs in
            key = ((idx[:, 0].long() * 256 + idx[:, 1]) * 256 + idx[:, 2]) * 256 + idx[:, 3]
            idx = idx[torch.argsort(key)]
        idx = idx.to(dev)
        feats = torch.randn(idx.shape[0], c, device=dev).half()
        for name, k, s in (("maxpool_k2s2", 2, 2), ("avgpool_k3s1", 3, 1)):
            res = P.igemm_pairs(idx, batch, [256] * 3, [k] * 3, [s] * 3, [0] * 3, [1] * 3, [0] * 3, False, False, True, False)
            pf, pb = res[2], res[3]
            n_out, kv = pf.shape[1], pf.shape[0]
            pairs = int((pf >= 0).sum())
            n_in = int(idx.shape[0])
            # gathered: every (pair, row) read counted (a 3^3 window re-reads rows out of L2);
            # compulsory: every input row once + table + stored rows, what has to cross the HBM interface
            fwd_gathered = pairs * c * 2 + n_out * c * 2 + kv * n_out * 4
            fwd_bytes = n_in * c * 2 + n_out * c * 2 + kv * n_out * 4
            if name.startswith("max"):
                out = PL.maxpool_forward(feats, pf, n_out)
                g = torch.randn_like(out)
                emit(name + "_fwd", timed(lambda: PL.maxpool_forward(feats, pf, n_out), iters), fwd_bytes,
                     voxels=n_in, n_out=n_out, pairs=pairs, voxel_order=args.voxel_order, bytes="compulsory",
                     gathered_bytes=fwd_gathered)
                # features + output + output gradient read, input gradient written, table
                bwd_bytes = n_in * c * 2 * 2 + n_out * c * 2 * 2 + kv * n_in * 4
                emit(name + "_bwd", timed(lambda: PL.maxpool_backward(feats, out, g, pb), iters), bwd_bytes,
                     bytes="compulsory", gathered_bytes=n_in * c * 2 * 2 + pairs * c * 2 * 2 + kv * n_in * 4)
            else:
                out, cnt = PL.avgpool_forward(feats, pf, n_out)
                g = torch.randn_like(out)
                emit(name + "_fwd", timed(lambda: PL.avgpool_forward(feats, pf, n_out), iters), fwd_bytes + 4 * n_out,
                     voxels=n_in, n_out=n_out, pairs=pairs, voxel_order=args.voxel_order, bytes="compulsory",
                     gathered_bytes=fwd_gathered + 4 * n_out)
                bwd_bytes = n_in * c * 2 + n_out * (c * 2 + 4) + kv * n_in * 4
                emit(name + "_bwd", timed(lambda: PL.avgpool_backward(g, pb, cnt), iters), bwd_bytes, bytes="compulsory",
                     gathered_bytes=n_in * c * 2 + pairs * (c * 2 + 4) + kv * n_in * 4)
    elif args.op == "dense":
        # the step after the backbone: 8 samples, 128 channels, BEV volume [2, 200, 176], 60k rows per sample
        import spconv_triton_b200.pytorch as sp
        from spconv_triton_b200.scenes import uniform_batch

        batch, shape, c = 8, [2, 200, 176], 128
        idx = torch.from_numpy(uniform_batch(5, batch, 40000, tuple(shape))).to(dev)
        key = ((idx[:, 0].long() * shape[0] + idx[:, 1]) * shape[1] + idx[:, 2]) * shape[2] + idx[:, 3]
        idx = idx[torch.argsort(key)]  # the order a rulebook emits
        feats = torch.randn(idx.shape[0], c, device=dev).half()
        x = sp.SparseConvTensor(feats, idx, shape, batch)
        vol = batch * shape[0] * shape[1] * shape[2]
        nbytes = vol * c * 2 + 2 * idx.shape[0] * c * 2 + idx.shape[0] * 16

        def torch_dense():
            res = torch.zeros([batch, *shape, c], dtype=feats.dtype, device=dev)
            il = idx.long()
            res[il[:, 0], il[:, 1], il[:, 2], il[:, 3]] = feats
            return res.permute(0, 4, 1, 2, 3).contiguous()

        emit("dense_channels_first", timed(lambda: x.dense(), iters), nbytes, rows=int(idx.shape[0]), dense_elems=vol * c,
             torch_definition_ms=timed(torch_dense, iters))
    elif args.op == "global_pool":
        # classification head: per-sample max / mean over 4 x 100k rows of 128 fp16 channels (batch order)
        import spconv_triton_b200.pytorch as sp
        from spconv_triton_b200.scenes import uniform_batch

        batch, shape, c = 4, [41, 400, 352], 128
        idx = torch.from_numpy(uniform_batch(21, batch, 100000, tuple(shape))).to(dev)
        x = sp.SparseConvTensor(torch.randn(idx.shape[0], c, device=dev).half(), idx, shape, batch)
        n = int(idx.shape[0])
        gmax, gavg = sp.SparseGlobalMaxPool(), sp.SparseGlobalAvgPool()

        def torch_definition():
            # the reference's formulation: rows per sample, host read of the counts, one gather + max per sample
            b = idx[:, 0].long()
            counts = torch.bincount(b, minlength=batch).cpu().numpy()
            order = torch.argsort(b, stable=True)
            res, start = [], 0
            for s in range(batch):
                res.append(torch.max(x.features[order[start:start + counts[s]]], dim=0)[0])
                start += counts[s]
            return torch.stack(res)

        emit("global_max_pool_400k_c128", timed(lambda: gmax(x), iters), n * c * 2 + n * 4, rows=n,
             torch_definition_ms=timed(torch_definition, iters))
        emit("global_avg_pool_400k_c128", timed(lambda: gavg(x), iters), n * 32 + n * 4, rows=n)
    elif args.op == "sparse_add":
        # the residual join of two branches with different voxel sets: 2 x 400k rows of 64 fp16 channels, 4 samples
        import spconv_triton_b200.pytorch as sp
        from spconv_triton_b200.scenes import uniform_batch

        batch, shape, c = 4, [41, 400, 352], 64
        tens = []
        for seed in (11, 12):
            idx = torch.from_numpy(uniform_batch(seed, batch, 100000, tuple(shape))).to(dev)
            tens.append(sp.SparseConvTensor(torch.randn(idx.shape[0], c, device=dev).half(), idx, shape, batch))
        out = sp.functional.sparse_add_hash_based(*tens)
        n_in, n_out = sum(int(t.indices.shape[0]) for t in tens), int(out.indices.shape[0])
        # read features + coordinates, write the union (read-modify-write of the second operand's rows)
        nbytes = n_in * (c * 2 + 16) + n_out * (c * 2 + 16) + int(tens[1].indices.shape[0]) * c * 2

        def torch_definition():
            # the reference's formulation (sort-based table): unique of the linear coordinates + index_add
            lin = [((t.indices[:, 0].long() * shape[0] + t.indices[:, 1]) * shape[1] + t.indices[:, 2]) * shape[2]
                   + t.indices[:, 3] for t in tens]
            uniq, inv = torch.unique(torch.cat(lin), return_inverse=True)
            res = torch.zeros([uniq.shape[0], c], dtype=tens[0].features.dtype, device=dev)
            ind = torch.zeros([uniq.shape[0], 4], dtype=torch.int32, device=dev)
            start = 0
            for t in tens:
                rows = inv[start:start + t.indices.shape[0]]
                start += t.indices.shape[0]
                res[rows] += t.features
                ind[rows] = t.indices
            return res, ind

        emit("sparse_add_hash_based_2x400k_c64", timed(lambda: sp.functional.sparse_add_hash_based(*tens), iters), nbytes,
             rows_in=n_in, rows_out=n_out, torch_definition_ms=timed(torch_definition, iters))
    elif args.op == "from_dense":
        # a BEV feature map back to sparse rows: [8, 200, 176, 128] fp16 channels-last, 12 % of the cells occupied
        import spconv_triton_b200.pytorch as sp

        g = torch.Generator().manual_seed(4)
        keep = (torch.rand(8, 200, 176, 1, generator=g) < 0.12).to(dev)
        x = (torch.randn(8, 200, 176, 128, device=dev) * keep).half()
        t = sp.SparseConvTensor.from_dense(x)
        rows, cells = int(t.indices.shape[0]), 8 * 200 * 176
        nbytes = cells * 128 * 2 + cells * 8 + rows * (12 + 2 * 128 * 2)

        def torch_definition():
            s_ = x.to_sparse(x.ndim - 1)
            return s_.values(), s_.indices().permute(1, 0).contiguous().int()

        emit("from_dense_8x200x176_c128", timed(lambda: sp.SparseConvTensor.from_dense(x), iters), nbytes, rows=rows,
             cells=cells, torch_definition_ms=timed(torch_definition, iters))
    elif args.op == "voxelize":
        # the step before the backbone: 8 LiDAR sweeps of 150k points -> voxels of 0.16 x 0.16 x 0.2 m
        from spconv_triton_b200.pytorch.utils import PointToVoxel

        g = torch.Generator().manual_seed(1)
        n, f, maxpts, cap = 1_200_000, 4, 5, 800_000
        pts = torch.cat([torch.randn(n, 3, generator=g) * torch.tensor([18.0, 18.0, 0.9]), torch.rand(n, 1, generator=g)], 1)
        pts = pts.to(dev)
        p2v = PointToVoxel([0.16, 0.16, 0.2], [-35.2, -40.0, -3.0, 35.2, 40.0, 1.0], f, cap, maxpts, dev)
        vox, idx, npv, pcvid = p2v.generate_voxel_with_id(pts)
        m = int(idx.shape[0])
        stored = int(npv.sum())
        nbytes = n * f * 4 + cap * maxpts * f * 4 + stored * f * 4 + n * 8 + m * 16
        emit("voxelize_1.2M_points", timed(lambda: p2v.generate_voxel_with_id(pts), iters), nbytes, points=n,
             voxels=m, stored_points=stored, mpoints_per_s=None)
    elif args.op == "conv_subm":
        # the backbone's dominant layer type: SubMConv3d k3 at the geometry two stride-2 layers leave
        batch, shape = 4, list(GRID)
        idx = torch.from_numpy(lidar_like_batch(3, batch, (16000, 24000), tuple(GRID))).to(dev)
        for _ in range(2):
            r = P.igemm_pairs(idx, batch, shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, False, False)
            idx, shape = r[0], P.get_conv_output_size(shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3)
        r = P.igemm_pairs(idx, batch, shape, [3] * 3, [1] * 3, [1] * 3, [1] * 3, [0] * 3, True, False, True, False)
        pf, pb, maf, mab, pmf, pmb = r[2], r[3], r[6][0], r[6][0], r[4][0], r[4][0]
        n, kv = idx.shape[0], pf.shape[0]
        pairs = int((pf >= 0).sum())
        for c in (32, 64, 128):
            x = torch.randn(n, c, device=dev).half()
            w = (torch.randn(c, kv, c, device=dev) * 0.02).half()
            g = torch.randn(n, c, device=dev).half()
            flops = 2.0 * pairs * c * c
            nbytes = pairs * c * 2 + n * c * 2 + kv * n * 4 + kv * c * c * 2
            emit(f"subm_fwd_{c}_{c}", timed(lambda: G.conv_forward(x, w, pf, n, pair_mask=pmf, mask_argsort=maf), iters),
                 nbytes, flops, voxels=n, pairs=pairs)
            emit(f"subm_dgrad_{c}_{c}", timed(lambda: G.conv_backward_input(g, w, pb, n, pair_mask=pmb, mask_argsort=mab), iters),
                 nbytes, flops)
            emit(f"subm_wgrad_{c}_{c}", timed(lambda: G.conv_backward_weight(x, g, pf, (c, kv, c)), iters),
                 pairs * 2 * c * 2 + kv * n * 4, flops)
    else:
        batch = 4
        idx = torch.from_numpy(lidar_like_batch(100, batch, (120000, 120000), tuple(GRID))).to(dev)
        n_in = idx.shape[0]
        args_rb = (idx, batch, GRID, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, True, False)
        res = P.igemm_pairs(*args_rb)
        out_inds, _, pf, pb, pmf, pmb, maf, mab, _ = res
        n_out, kv = pf.shape[1], pf.shape[0]
        pairs = int((pf >= 0).sum())
        rb_bytes = n_in * 16 + n_out * 16 + kv * n_out * 4 + kv * n_in * 4 + 8 * n_out + 8 * n_in
        emit("rulebook_k3s2", timed(lambda: P.igemm_pairs(*args_rb), iters), rb_bytes, voxels=n_in, n_out=n_out, pairs=pairs)
        x = torch.randn(n_in, 64, device=dev).half()
        w = (torch.randn(128, kv, 64, device=dev) * 0.02).half()
        g = torch.randn(n_out, 128, device=dev).half()
        flops = 2.0 * pairs * 64 * 128
        emit("conv_fwd_64_128", timed(lambda: G.conv_forward(x, w, pf, n_out, pair_mask=pmf[0][:, 0], mask_argsort=maf[0]), iters),
             pairs * 64 * 2 + n_out * 128 * 2 + kv * n_out * 4, flops)
        emit("conv_dgrad_64_128", timed(lambda: G.conv_backward_input(g, w, pb, n_in, pair_mask=pmb[0][:, 0], mask_argsort=mab[0]), iters),
             pairs * 128 * 2 + n_in * 64 * 2 + kv * n_in * 4, flops)
        emit("conv_wgrad_64_128", timed(lambda: G.conv_backward_weight(x, g, pf, (128, kv, 64)), iters),
             pairs * (64 + 128) * 2 + kv * n_out * 4, flops)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-baseline-seconds", type=float, default=20.0)
    ap.add_argument("--op", default=None, choices=["pool", "conv_s2", "conv_subm", "conv_k5", "published", "published_reference",
                             "backbone_reference_gpu", "voxelize", "dense", "sparse_add", "global_pool", "from_dense"],
                    help="single-operator timings at the other configurations instead of the headline benchmark")
    ap.add_argument("--k5-voxels", type=int, default=400000, help="--op conv_k5: voxels per sample (4 samples)")
    ap.add_argument("--pool-voxels", type=int, default=400000, help="--op pool: voxels per sample (4 samples)")
    ap.add_argument("--in-flight", type=int, default=3,
                    help="independent steps in flight at a time, each issued by its own host thread and CUDA stream "
                         "(1 = one pass after the other); lowered to what the host cores of this rank allow")
    ap.add_argument("--no-train", action="store_true",
                    help="skip the training-step record (BASELINE configs[3]) that follows the headline measurement")
    ap.add_argument("--voxel-order", default="random", choices=["random", "sorted"],
                    help="--op pool: input voxel order (random = as a voxeliser emits them, sorted = as a previous layer's rulebook emits them)")
    args = ap.parse_args()
    if args.op is not None:
        run_op_bench(args)
        return
    if args.impl == "reference":
        args.steps = min(args.steps, 8)
        args.warmup = min(args.warmup, 1)
        run_reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    args.warmup = max(args.warmup, 3)
    # every pass in flight keeps a host thread waiting on the device (the reads of the output counts)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    if cores // world >= args.in_flight + 1:
        pass  # a core per pass in flight and one for the main thread: the waits may spin
    else:
        # fewer cores than waiting threads: the library's waits sleep instead of spinning (read by
        # the library at its first rulebook call), and the passes in flight still fit twice over
        os.environ["SPC_HOST_WAIT"] = "block"
        args.in_flight = max(1, min(args.in_flight, 2 * cores // world - 1))

    from spconv_triton_b200 import _lib
    import spconv_triton_b200.pytorch as sp

    lib = _lib.load()
    clocks = ClockSampler(local_rank)
    net = init_backbone(build_backbone()).half().eval().to(dev)
    scenes_host = [(i.pin_memory(), f.pin_memory()) for i, f in make_scenes(rank)]
    scenes_dev = [(i.to(dev), f.to(dev)) for i, f in scenes_host]
    voxels_per_scene = [int(i.shape[0]) for i, _ in scenes_host]
    prof = GemmProfiler()
    prof.install()
    generating = []
    for L in LAYERS:
        if L["key"] not in generating:
            generating.append(L["key"])
    rb_prof = RulebookProfiler(generating)
    rb_prof.install()

    def forward(idx, feats, scene=0):
        prof.scene, prof.call = scene, 0
        with torch.no_grad():
            return net(sp.SparseConvTensor(feats, idx, GRID, BATCH))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident arm: inputs already in HBM -------------------------------------
    from spconv_triton_b200 import constants as spc_constants

    # untimed, layer by layer from Python so that every GEMM call is seen: algorithmic pair
    # counts of every (scene, layer)
    native_sequence = spc_constants.SPCONV_NATIVE_SEQUENCE
    spc_constants.SPCONV_NATIVE_SEQUENCE = False
    prof.enabled = prof.count_pairs = True
    for s in range(N_SCENES):
        out = forward(*scenes_dev[s], scene=s)
    prof.enabled = prof.count_pairs = False
    spc_constants.SPCONV_NATIVE_SEQUENCE = native_sequence
    # warm-up with the timed loop's own allocation pattern (each step's output is
    # released before the next step starts), over every scene, so that the caching
    # allocator makes no cudaMalloc inside the timed region
    for w in range(max(args.warmup, 3 * N_SCENES)):
        out = None
        out = forward(*scenes_dev[w % N_SCENES], scene=w % N_SCENES)
    # Consecutive steps are independent passes over different scenes.  A pass blocks its host thread
    # at every strided layer (the read of the output count), so the steps are issued by worker
    # threads, each on its own stream, with `--in-flight` passes in flight: the kernels that open
    # step s+1 then overlap the ones that close step s.
    import collections

    from spconv_triton_b200.parallel import PassPipeline

    pipe = PassPipeline(dev, depth=args.in_flight)

    def run_steps(n_steps, fn):
        """fn(s) for s in 0..n_steps-1 on the pipeline, at most `in_flight` at a time; results are
        dropped as they complete (so that their memory returns to the allocator); returns the last."""
        window, last = collections.deque(), None
        for s in range(n_steps):
            if len(window) == args.in_flight:
                last = window.popleft().result()
            window.append(pipe.submit(fn, s))
        while window:
            last = window.popleft().result()
        pipe.join()
        return last

    def resident_step(s):
        return forward(*scenes_dev[s % N_SCENES], scene=s % N_SCENES)

    run_steps(4 * args.in_flight + N_SCENES, resident_step)  # every worker's allocator pool sees the pattern
    # A cudaMalloc inside a timed region (the caching allocator growing a pool because the worker
    # threads interleaved differently than in the warm-up) synchronises the device and is not the
    # steady state: such a measurement is taken again, at most twice, and the count is reported.
    clocks.open_window()
    resident_attempts = 0
    while True:
        resident_attempts += 1
        barrier()
        launches0 = lib.spc_launch_count()
        mallocs0 = torch.cuda.memory_stats(dev).get("num_device_alloc", 0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = run_steps(args.steps, resident_step)
        e1.record()
        barrier()
        mallocs_resident = torch.cuda.memory_stats(dev).get("num_device_alloc", 0) - mallocs0
        launches = lib.spc_launch_count() - launches0
        if sum_over_ranks(mallocs_resident) == 0 or resident_attempts == 3:
            break
    dev_ms = max_over_ranks(e0.elapsed_time(e1))
    voxels = sum(voxels_per_scene[s % N_SCENES] for s in range(args.steps))
    total_voxels = sum_over_ranks(voxels)
    value = total_voxels / (dev_ms * 1e-3) / 1e6

    # ---- end-to-end arm: pinned host buffers in, the output tensor (features + indices) out ----
    # Every step copies its inputs from pinned host memory, runs the forward and copies the whole
    # output tensor (features + indices) back to pinned host memory.  The copy back runs on its own
    # stream into one of two host buffers, so that step s+1 computes while the result of step s
    # crosses PCIe; a buffer is handed out again only after its copy has completed.
    h2d = int(np.mean([i.numel() * 4 + f.numel() * 2 for i, f in scenes_host]))
    max_rows = int(out.features.shape[0] * 1.5) + 1024
    n_slots = 2 * args.in_flight
    host_out = [(torch.empty((max_rows, out.features.shape[1]), dtype=out.features.dtype).pin_memory(),
                 torch.empty((max_rows, 4), dtype=torch.int32).pin_memory()) for _ in range(n_slots)]
    landed = [None] * n_slots
    in_transit = [None] * n_slots  # the output tensors whose copy to the host may still be running
    copy_stream = torch.cuda.Stream(device=dev)
    d2h_bytes = []

    def e2e_step(s):
        # runs on a worker thread, under that worker's stream
        slot = s % n_slots
        if landed[slot] is not None:
            landed[slot].synchronize()  # the result that used this buffer has arrived (and been consumed)
            in_transit[slot] = None     # its device memory goes back to the allocator only now
        idx_h, feats_h = scenes_host[s % N_SCENES]
        idx = idx_h.to(dev, non_blocking=True)
        feats = feats_h.to(dev, non_blocking=True)
        o = forward(idx, feats)
        n = o.features.shape[0]
        computed = torch.cuda.Event()
        computed.record()
        copy_stream.wait_event(computed)
        with torch.cuda.stream(copy_stream):
            host_out[slot][0][:n].copy_(o.features, non_blocking=True)
            host_out[slot][1][:n].copy_(o.indices, non_blocking=True)
            done = torch.cuda.Event()
            done.record(copy_stream)
        landed[slot], in_transit[slot] = done, o
        d2h_bytes.append(n * (o.features.shape[1] * o.features.element_size() + 16))
        return None

    def e2e_drain():
        torch.cuda.current_stream().wait_stream(copy_stream)

    run_steps(max(args.warmup, 4 * n_slots), e2e_step)  # buffers, allocator pools and copy stream in steady state
    e2e_drain()
    d2h_bytes.clear()
    # what the link gives a plain device-to-host copy of one result's size (pinned memory, copy stream)
    torch.cuda.synchronize()
    n_probe = min(max_rows, out.features.shape[0])
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(copy_stream):
        p0.record(copy_stream)
        for _ in range(4):
            host_out[0][0][:n_probe].copy_(out.features[:n_probe], non_blocking=True)
        p1.record(copy_stream)
    copy_stream.synchronize()
    d2h_gbps = 4 * n_probe * out.features.shape[1] * out.features.element_size() / (p0.elapsed_time(p1) * 1e-3) / 1e9
    e2e_attempts = 0  # same rule as for the device-resident arm
    while True:
        e2e_attempts += 1
        barrier()
        mallocs1 = torch.cuda.memory_stats(dev).get("num_device_alloc", 0)
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record()
        run_steps(args.steps, e2e_step)
        e2e_drain()  # the last results have to be on the host before the clock stops
        e3.record()
        barrier()
        mallocs_e2e = torch.cuda.memory_stats(dev).get("num_device_alloc", 0) - mallocs1
        if sum_over_ranks(mallocs_e2e) == 0 or e2e_attempts == 3:
            break
        d2h_bytes.clear()
    clocks.close_window()
    clocks.stop()
    e2e_ms = max_over_ranks(e2.elapsed_time(e3))
    e2e_value = total_voxels / (e2e_ms * 1e-3) / 1e6

    # ---- the kernels alone: the same steps once more with the rulebook run-ahead off, so that no
    # rulebook kernel shares the SMs with the GEMM launches (and no GEMM with the rulebooks) that
    # the events bracket -------------------------------------------------------------------------
    runahead = spc_constants.SPCONV_RULEBOOK_RUNAHEAD
    spc_constants.SPCONV_RULEBOOK_RUNAHEAD = False  # also sends the pass through the modules one by one
    for w in range(N_SCENES):
        out = None
        out = forward(*scenes_dev[w % N_SCENES], scene=w % N_SCENES)
    prof.records.clear()
    prof.enabled = rb_prof.enabled = True
    torch.cuda.synchronize()
    ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ea.record()
    for s in range(args.steps):
        out = None
        out = forward(*scenes_dev[s % N_SCENES], scene=s % N_SCENES)
    eb.record()
    torch.cuda.synchronize()
    prof.enabled = rb_prof.enabled = False
    gemm = prof.summarize()
    rulebook_ms, rulebook_total_ms = rb_prof.summarize(args.steps)
    serial_ms = ea.elapsed_time(eb)
    spc_constants.SPCONV_RULEBOOK_RUNAHEAD = runahead

    # ---- footprint: shows the per-step working set exceeds L2 ------------------------------
    idict = out.indice_dict
    table_bytes = sum(d.pair_fwd.numel() * 4 + (d.pair_bwd.numel() * 4 if d.pair_bwd is not None else 0)
                      for d in idict.values())
    out = None

    # ---- BASELINE configs[3]: the training step with the gradient all-reduce ---------------
    train = None
    if not args.no_train:
        torch.cuda.empty_cache()
        train = run_train_arm(dev, rank, world, steps=max(3, min(args.steps, 10)), warmup=10)

    if rank != 0:
        clocks.summary()
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    achieved_tflops = gemm["flops"] / (gemm["ms"] * 1e-3) / 1e12 if gemm["ms"] else 0.0
    compulsory_gbs = gemm["compulsory"] / (gemm["ms"] * 1e-3) / 1e9 if gemm["ms"] else 0.0
    gathered_gbs = gemm["bytes"] / (gemm["ms"] * 1e-3) / 1e9 if gemm["ms"] else 0.0
    traffic, traffic_source = captured_gemm_traffic()

    cpu_baseline = None
    if world == 1:
        cpu_baseline = cpu_baseline_sample(net, args.cpu_baseline_seconds)

    line = {
        "metric": "voxelnet_backbone_fwd_mvoxels_per_s", "value": value, "unit": "Mvoxels/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {
            "workload": "BASELINE configs[2]: VoxelNet-style sparse middle encoder, fp16 inference, "
                        "grid [41,1600,1408], batch 8 per GPU, 16k-24k voxels/sample, rulebooks rebuilt every step",
            "voxels_per_step": int(np.mean(voxels_per_scene)), "scenes": N_SCENES,
            "l2": f"inputs larger than L2: rulebook tables of one step hold {table_bytes / 1e6:.0f} MB "
                  "and scenes rotate every step",
            "parallelism": f"replicas x{world} (sharded by sample, no collective)",
            "in_flight": f"{args.in_flight} steps in flight (independent passes over different scenes, issued by "
                         f"{args.in_flight} host threads on their own streams); --in-flight 1 = one pass after the other",
        },
        "e2e": {"value": e2e_value, "unit": "Mvoxels/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": int(np.mean(d2h_bytes)), "ms_per_step": e2e_ms / args.steps,
                "d2h_link_GBps": d2h_gbps,
                "result": "output features and indices copied to pinned host memory every step, on a copy stream, "
                          "double-buffered (step s+1 computes while the result of step s crosses PCIe)",
                "in_flight": args.in_flight},
        "gpu_launches": int(launches),
        "allocator": {"device_mallocs_in_timed_region": int(mallocs_resident),
                      "device_mallocs_in_e2e_timed_region": int(mallocs_e2e),
                      "measurements": resident_attempts, "e2e_measurements": e2e_attempts},
        "clocks": clocks.summary(),
        "rulebook_ms": {"per_indice_key": rulebook_ms, "per_step": rulebook_total_ms,
                        "timing": "CUDA events around each rulebook generation, run-ahead off (host read of the "
                                  "output count included)"},
        "roofline": {
            "kernel": "gather-GEMM forward (every launch of the timed steps, aggregated)",
            "timing": "CUDA events around each launch on its stream, in a repeat of the timed steps with the "
                      "rulebook run-ahead off so that the kernel runs alone",
            "bound": "tensor", "achieved": achieved_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
            "frac": achieved_tflops / tensor_peak if tensor_peak else None,
            "traffic": traffic, "traffic_source": traffic_source,
            "flops_per_launch": gemm["flops"] / gemm["launches"] if gemm["launches"] else None,
            "peak_kind": peak_kind + " (bf16 cuBLAS burst)",
            "launches": gemm["launches"], "avg_launch_ms": gemm["avg_ms"],
            "share_of_step": gemm["ms"] / serial_ms if serial_ms else None,
            "serial_ms_per_step": serial_ms / args.steps,
            "rulebook_runahead": bool(runahead), "native_sequence": bool(native_sequence),
            "per_layer": gemm["layers"],
            "hbm": {"peak": hbm_peak, "unit": "GB/s",
                    "compulsory_bytes_per_launch": gemm["compulsory"] / gemm["launches"] if gemm["launches"] else None,
                    "compulsory_GBps": compulsory_gbs, "compulsory_frac": compulsory_gbs / hbm_peak if hbm_peak else None,
                    "gathered_bytes_per_launch": gemm["bytes"] / gemm["launches"] if gemm["launches"] else None,
                    "gathered_GBps": gathered_gbs,
                    "note": "gathered = every (pair, row) read counted, mostly L2 hits; compulsory = every input "
                            "row once + table + stored rows + weights"},
        },
        "cpu_baseline": cpu_baseline,
    }
    if train is not None:
        line["train"] = train
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline_sample(net, budget_s):
    """The oracle port on the host cores over single samples of the workload,
    repeated until about ``budget_s`` seconds of CPU work are spent."""
    from oracle.backbone import run_backbone

    if budget_s <= 0:
        return None
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    params = oracle_params(net)
    scenes = make_scenes(0, n_scenes=2, batch=1)
    spent, voxels, runs = 0.0, 0, 0
    while spent < budget_s and runs < 8:
        idx, feats = scenes[runs % len(scenes)]
        t0 = time.perf_counter()
        run_backbone(LAYERS, params, idx.numpy(), feats.float(), GRID, 1, acc_dtype=torch.float32)
        spent += time.perf_counter() - t0
        voxels += idx.shape[0]
        runs += 1
    return {"value": voxels / spent / 1e6, "unit": "Mvoxels/s", "cores": cores, "kind": "port",
            "sample": f"{runs} single-sample forwards ({voxels} voxels, {spent:.1f} s) of the same backbone, "
                      "numpy rulebook + torch CPU fp32 gather-matmul"}


if __name__ == "__main__":
    main()
