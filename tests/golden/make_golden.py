"""Generate the golden vectors under tests/golden/ from the reference itself.

Run once in a container that has the reference checkout (read-only) at
$SPCONV_REFERENCE_ROOT:

    python tests/golden/make_golden.py

Two kinds of vectors are written:

1. ``ref_ops.npz`` -- outputs of the reference's own hot-path functions
   (``_impl.pairs.igemm_pairs`` / ``native_pairs`` / ``native_pair_to_tables``,
   ``_impl.gemm.conv_forward`` / ``conv_backward_input`` /
   ``conv_backward_weight``, ``_impl.pool.*``) on small seeded inputs.  The
   reference is Triton-only, so its kernels are executed on CPU tensors by
   Triton's interpreter (TRITON_INTERPRET=1) with the autotuner pinned to each
   kernel's first configuration (all configurations are numerically equivalent
   by the reference's own contract).
2. ``ref_frozen.pt`` -- the hot-path cases of the reference's frozen golden
   files (tests/data/golden_net.pt, golden_misc.pt:seq2d_mixed,
   golden_ext_pool.pt, golden_proto.pt), re-saved unchanged so the test-suite
   does not need the reference checkout at run time.

Nothing here is imported by the product or by the tests; the tests only read
the files it writes.
"""

import json
import os
import sys
from pathlib import Path

REF = os.environ["SPCONV_REFERENCE_ROOT"]  # the read-only reference checkout
OUT = Path(__file__).parent

os.environ["TRITON_INTERPRET"] = "1"
import importlib.metadata as _md  # noqa: E402

_orig_version = _md.version
_md.version = lambda n: "1.0.0" if n == "spconv-triton" else _orig_version(n)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402,F401
from triton.runtime import autotuner as _at  # noqa: E402


def _run_first_config(self, *args, **kwargs):
    cfg = self.configs[0]
    return self.fn.run(*args, **{**kwargs, **cfg.all_kwargs()})


_at.Autotuner.run = _run_first_config
torch.Tensor.is_cuda = property(lambda self: True)
sys.path.insert(0, REF)

from spconv_triton.pytorch._impl import gemm as ref_gemm  # noqa: E402
from spconv_triton.pytorch._impl import pairs as ref_pairs  # noqa: E402
from spconv_triton.pytorch._impl import pool as ref_pool  # noqa: E402

ref_gemm._multiprocessor_count = lambda device: 16


def unique_coords(rng, n, batch, shape):
    """n unique (batch, *coords) rows, batch-major order, int32."""
    vol = int(np.prod(shape))
    per = [n // batch + (1 if b < n % batch else 0) for b in range(batch)]
    rows = []
    for b, m in enumerate(per):
        lin = np.sort(rng.choice(vol, size=m, replace=False))
        c = np.stack(np.unravel_index(lin, shape), axis=1)
        rows.append(np.concatenate([np.full((m, 1), b), c], axis=1))
    out = np.concatenate(rows, 0).astype(np.int32)
    # shuffle rows inside the whole tensor so row order is not coordinate order
    return out[rng.permutation(out.shape[0])]


def E(x, n):
    return [x] * n if isinstance(x, int) else list(x)


# name, ndim, shape, batch, N, ksize, stride, pad, dil, out_pad, subm, transpose, extra
RULEBOOK_CASES = [
    ("subm3d_k3", [16, 16, 16], 2, 400, 3, 1, 1, 1, 0, True, False, {}),
    ("subm3d_k3_cfg1", [64, 64, 64], 1, 2000, 3, 1, 1, 1, 0, True, False, {}),
    ("subm3d_k3_eval", [12, 14, 10], 3, 300, 3, 1, 0, 1, 0, True, False, {"is_train": False}),
    ("conv3d_k3s2p1", [16, 16, 16], 2, 400, 3, 2, 1, 1, 0, False, False, {}),
    ("conv3d_k2s2", [16, 18, 14], 2, 350, 2, 2, 0, 1, 0, False, False, {}),
    ("conv3d_k3s1d2p2", [10, 10, 10], 2, 200, 3, 1, 2, 2, 0, False, False, {}),
    ("conv3d_k1s2", [12, 12, 12], 2, 200, 1, 2, 0, 1, 0, False, False, {}),
    ("convT3d_k3s2p1op1", [8, 8, 8], 2, 120, 3, 2, 1, 1, 1, False, True, {}),
    ("subm2d_k3d2", [24, 20], 3, 300, 3, 1, 0, 2, 0, True, False, {}),
    ("conv2d_k32s21p10", [24, 20], 3, 300, [3, 2], [2, 1], [1, 0], 1, 0, False, False, {}),
    ("conv1d_k3s2", [64], 4, 120, 3, 2, 1, 1, 0, False, False, {}),
    ("subm4d_k3", [8, 8, 8, 8], 2, 150, 3, 1, 1, 1, 0, True, False, {}),
    ("conv3d_k5s1_kv125", [8, 8, 8], 1, 60, 5, 1, 0, 1, 0, False, False, {}),
    ("subm3d_k5_kv125", [10, 10, 10], 2, 150, 5, 1, 2, 1, 0, True, False, {}),
    ("conv3d_k3s2p1_split", [16, 16, 16], 2, 300, 3, 2, 1, 1, 0, False, False, {"is_mask_split": True}),
    ("conv3d_k3s2p1_nosort", [16, 16, 16], 2, 300, 3, 2, 1, 1, 0, False, False, {"do_sort": False}),
    ("conv3d_k3s2p1_bound", [16, 16, 16], 2, 300, 3, 2, 1, 1, 0, False, False, {"num_out_act_bound": 150}),
    ("conv3d_k3s2p1_eval", [16, 16, 16], 2, 300, 3, 2, 1, 1, 0, False, False, {"is_train": False}),
]


def gen_rulebooks(store):
    specs = {}
    for ci, (name, shape, batch, n, k, s, p, d, op, subm, tr, extra) in enumerate(RULEBOOK_CASES):
        ndim = len(shape)
        rng = np.random.default_rng(1000 + ci)
        idx = unique_coords(rng, n, batch, shape)
        args = dict(batch_size=batch, spatial_shape=list(shape), ksize=E(k, ndim), stride=E(s, ndim),
                    padding=E(p, ndim), dilation=E(d, ndim), out_padding=E(op, ndim),
                    subm=subm, transpose=tr)
        ig = dict(is_train=extra.get("is_train", True), is_mask_split=extra.get("is_mask_split", False),
                  do_sort=extra.get("do_sort", True), num_out_act_bound=extra.get("num_out_act_bound", -1))
        t_idx = torch.from_numpy(idx)
        res = ref_pairs.igemm_pairs(t_idx, args["batch_size"], args["spatial_shape"], args["ksize"],
                                    args["stride"], args["padding"], args["dilation"], args["out_padding"],
                                    subm, tr, ig["is_train"], ig["is_mask_split"], ig["do_sort"],
                                    ig["num_out_act_bound"])
        out_inds, npl, pf, pb, pmf, pmb, maf, mab, masks = res
        pre = f"rb/{name}/"
        store[pre + "indices"] = idx
        store[pre + "ig_out_inds"] = out_inds.numpy()
        store[pre + "ig_npl"] = npl.numpy()
        store[pre + "ig_pair_fwd"] = pf.numpy()
        store[pre + "ig_pair_bwd"] = pb.numpy() if pb.numel() else np.zeros((0,), np.int32)
        for i, t in enumerate(pmf):
            store[pre + f"ig_pm_fwd{i}"] = t.numpy()
        for i, t in enumerate(pmb):
            store[pre + f"ig_pm_bwd{i}"] = t.numpy()
        for i, t in enumerate(maf):
            store[pre + f"ig_ma_fwd{i}"] = t.numpy()
        for i, t in enumerate(mab):
            store[pre + f"ig_ma_bwd{i}"] = t.numpy()
        store[pre + "ig_masks"] = np.concatenate([np.asarray(m, dtype=np.uint32) for m in masks])
        if ig["is_mask_split"] or ig["num_out_act_bound"] > 0 or not ig["do_sort"]:
            pass
        else:
            o2, pair, npl2 = ref_pairs.native_pairs(t_idx, args["batch_size"], args["spatial_shape"],
                                                    args["ksize"], args["stride"], args["padding"],
                                                    args["dilation"], args["out_padding"], subm, tr)
            store[pre + "nat_out_inds"] = o2.numpy()
            store[pre + "nat_pair"] = pair.numpy()
            store[pre + "nat_npl"] = npl2.numpy()
            for inverse in (False, True):
                n_in, n_out = idx.shape[0], o2.shape[0]
                if inverse:
                    n_in, n_out = n_out, n_in
                p2 = pair.clone()  # memoisation lives on the tensor object
                tf, tb = ref_pairs.native_pair_to_tables(p2, npl2, n_in, n_out, inverse)
                store[pre + f"nat_tables_fwd_inv{int(inverse)}"] = tf.numpy()
                store[pre + f"nat_tables_bwd_inv{int(inverse)}"] = tb.numpy()
        specs[name] = dict(args=args, igemm=ig)
        print("rulebook", name, "n_out", int(out_inds.shape[0]), flush=True)
    return specs


# name, rulebook case, C_in, C_out, dtype, bias, masked
FEATURE_CASES = [
    ("subm_cfg1_f32", "subm3d_k3_cfg1", 16, 16, "float32", True, True),
    ("subm_f32", "subm3d_k3", 8, 12, "float32", True, True),
    ("subm_f16", "subm3d_k3", 16, 32, "float16", False, True),
    ("conv_s2_f32", "conv3d_k3s2p1", 6, 10, "float32", True, True),
    ("conv_s2_f16", "conv3d_k3s2p1", 32, 16, "float16", True, True),
    ("convT_f32", "convT3d_k3s2p1op1", 5, 7, "float32", False, True),
    ("conv2d_f32", "conv2d_k32s21p10", 9, 4, "float32", True, True),
    ("subm4d_f32", "subm4d_k3", 4, 4, "float32", False, False),
    ("kv125_f32", "conv3d_k5s1_kv125", 3, 5, "float32", True, False),
]

POOL_CASES = [
    ("max_k2s2_f32", "conv3d_k2s2", 7, "float32"),
    ("max_k3s2_f16", "conv3d_k3s2p1", 16, "float16"),
    ("max_subm_f32", "subm3d_k3", 5, "float32"),
    ("max_k3s2_f64", "conv3d_k3s2p1", 3, "float64"),
    ("avg_k2s2_f32", "conv3d_k2s2", 7, "float32"),
    ("avg_k3s2_f16", "conv3d_k3s2p1", 16, "float16"),
    ("avg_subm_f32", "subm3d_k3", 5, "float32"),
]


def gen_features(store):
    specs = {}
    for ci, (name, rb, cin, cout, dt, use_bias, masked) in enumerate(FEATURE_CASES):
        g = torch.Generator().manual_seed(2000 + ci)
        dtype = getattr(torch, dt)
        pre_rb = f"rb/{rb}/"
        pf = torch.from_numpy(store[pre_rb + "ig_pair_fwd"])
        pb = torch.from_numpy(store[pre_rb + "ig_pair_bwd"])
        n_in = store[pre_rb + "indices"].shape[0]
        n_out = pf.shape[1]
        kv = pf.shape[0]
        feats = torch.randn(n_in, cin, generator=g).to(dtype)
        w = (torch.randn(cout, kv, cin, generator=g) / (kv * cin) ** 0.5).to(dtype)
        bias = torch.randn(cout, generator=g).to(dtype) if use_bias else None
        gout = torch.randn(n_out, cout, generator=g).to(dtype)
        pm = ma = pmb = mab = None
        if masked and kv <= 32:
            pm = torch.from_numpy(store[pre_rb + "ig_pm_fwd0"])[:, 0].contiguous()
            ma = torch.from_numpy(store[pre_rb + "ig_ma_fwd0"])
            if (pre_rb + "ig_pm_bwd0") in store:
                pmb = torch.from_numpy(store[pre_rb + "ig_pm_bwd0"])[:, 0].contiguous()
                mab = torch.from_numpy(store[pre_rb + "ig_ma_bwd0"])
        out = ref_gemm.conv_forward(feats, w, pf, n_out, bias=bias, pair_mask=pm, mask_argsort=ma)
        din = ref_gemm.conv_backward_input(gout, w, pb, n_in, pair_mask=pmb, mask_argsort=mab)
        dw = ref_gemm.conv_backward_weight(feats, gout, pf, w.shape)
        pre = f"ft/{name}/"
        for key, t in dict(features=feats, weight=w, grad_out=gout, out=out, din=din, dw=dw).items():
            store[pre + key] = t.numpy()
        if bias is not None:
            store[pre + "bias"] = bias.numpy()
        specs[name] = dict(rulebook=rb, dtype=dt)
        print("features", name, flush=True)
    for ci, (name, rb, c, dt) in enumerate(POOL_CASES):
        g = torch.Generator().manual_seed(3000 + ci)
        dtype = getattr(torch, dt)
        pre_rb = f"rb/{rb}/"
        pf = torch.from_numpy(store[pre_rb + "ig_pair_fwd"])
        pb = torch.from_numpy(store[pre_rb + "ig_pair_bwd"])
        n_in = store[pre_rb + "indices"].shape[0]
        n_out = pf.shape[1]
        # a coarse value grid makes ties (max-pool backward) and all-negative windows likely
        feats = (torch.randint(-6, 4, (n_in, c), generator=g).to(torch.float32) * 0.25).to(dtype)
        gout = torch.randn(n_out, c, generator=g).to(dtype)
        pre = f"pl/{name}/"
        store[pre + "features"] = feats.numpy()
        store[pre + "grad_out"] = gout.numpy()
        if name.startswith("max"):
            out = ref_pool.maxpool_forward(feats, pf, n_out)
            din = ref_pool.maxpool_backward(feats, out, gout, pb)
        else:
            out, cnt = ref_pool.avgpool_forward(feats, pf, n_out)
            din = ref_pool.avgpool_backward(gout, pb, cnt)
            store[pre + "count"] = cnt.numpy()
        store[pre + "out"] = out.numpy()
        store[pre + "din"] = din.numpy()
        specs[name] = dict(rulebook=rb, dtype=dt)
        print("pool", name, flush=True)
    return specs


def extract_frozen():
    data = Path(REF) / "tests" / "data"
    keep = {
        "golden_net.pt": None,
        "golden_ext_pool.pt": None,
        "golden_misc.pt": {"seq2d_mixed"},
        "golden_proto.pt": None,
    }
    out = {}
    for fname, ids in keep.items():
        d = torch.load(data / fname, map_location="cpu", weights_only=False)
        out[fname] = [c for c in d["cases"] if ids is None or c["id"] in ids]
    torch.save(out, OUT / "ref_frozen.pt")
    print("frozen cases:", {k: [c["id"] for c in v] for k, v in out.items()})


def main():
    store = {}
    rb_specs = gen_rulebooks(store)
    ft_specs = gen_features(store)
    store["specs_json"] = np.frombuffer(
        json.dumps(dict(rulebooks=rb_specs, features=ft_specs)).encode(), dtype=np.uint8)
    np.savez_compressed(OUT / "ref_ops.npz", **store)
    extract_frozen()


if __name__ == "__main__":
    main()
