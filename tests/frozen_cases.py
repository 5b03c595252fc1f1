"""Runner for the reference's frozen golden cases (tests/golden/ref_frozen.pt):
builds the layers a case describes from this package, runs forward and
backward, and compares with the stored expectations (canonical order =
ascending batch-major linear coordinate, tolerances stored with each case)."""

from pathlib import Path

import torch

GOLDEN = Path(__file__).parent / "golden"
_cache = {}


def frozen(file, case_id):
    if "d" not in _cache:
        _cache["d"] = torch.load(GOLDEN / "ref_frozen.pt", map_location="cpu", weights_only=False)
    for c in _cache["d"][file]:
        if c["id"] == case_id:
            return c
    raise KeyError(case_id)


def frozen_ids(file):
    if "d" not in _cache:
        _cache["d"] = torch.load(GOLDEN / "ref_frozen.pt", map_location="cpu", weights_only=False)
    return [c["id"] for c in _cache["d"][file]]


def canonical_order(indices, spatial_shape):
    lin = indices[:, 0].long()
    for i, s in enumerate(spatial_shape):
        lin = lin * int(s) + indices[:, i + 1].long()
    return torch.argsort(lin)


def assert_close(actual, expected, atol, what):
    a = actual.detach().cpu().double()
    e = expected.detach().cpu().double()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} != {tuple(e.shape)}"
    if a.numel():
        err = (a - e).abs().max().item()
        assert err <= atol, f"{what}: max abs err {err:.3e} > atol {atol:.3e} (ref max {e.abs().max().item():.3e})"


def build_layer(sp, spec, dtype, device):
    from spconv_triton_b200.compat import tv
    from spconv_triton_b200.core import ConvAlgo

    if spec["cls"] == "SparseSequential":
        return sp.SparseSequential(*[build_layer(sp, c, dtype, device) for c in spec["children"]])
    if spec["cls"].startswith("nn."):
        cls = getattr(torch.nn, spec["cls"][3:])
    else:
        from spconv_triton_b200.pytorch import conv, pool

        cls = getattr(sp, spec["cls"], None) or getattr(conv, spec["cls"], None) or getattr(pool, spec["cls"])
    ctor = dict(spec["ctor"])
    if isinstance(ctor.get("act_type"), str):
        ctor["act_type"] = getattr(tv.gemm.Activation, ctor["act_type"])
    if isinstance(ctor.get("algo"), str):
        ctor["algo"] = getattr(ConvAlgo, ctor["algo"])
    layer = cls(**ctor).to(device)
    if dtype == torch.float16:
        layer = layer.half()
    with torch.no_grad():
        for name, value in (spec.get("params") or {}).items():
            if value is not None:
                getattr(layer, name).copy_(value.to(device))
    return layer


def check_sparse_output(out, expect, dtype, what):
    assert list(out.spatial_shape) == list(expect["out_spatial_shape"]), what
    order = canonical_order(out.indices.cpu(), out.spatial_shape)
    assert torch.equal(out.indices.cpu()[order], expect["out_indices"]), f"{what}: out indices differ"
    assert out.features.dtype == dtype, f"{what}: dtype {out.features.dtype}"
    assert_close(out.features.detach().cpu()[order], expect["out_features"], expect["atol_out"], f"{what}: out")
    return order


def run_pipeline_case(sp, case, device):
    dtype = getattr(torch, case["dtype"])
    training = bool(case["training"])
    layers = [build_layer(sp, s, dtype, device) for s in case["layers"]]
    for layer in layers:
        layer.train(training)
    inp = case["input"]
    feats = inp["features"].to(device).clone().requires_grad_(training)
    x = sp.SparseConvTensor(feats, inp["indices"].to(device), list(inp["spatial_shape"]), int(inp["batch_size"]))
    with torch.set_grad_enabled(training):
        out = x
        for layer in layers:
            out = layer(out)
    expect = case["expect"]
    order = check_sparse_output(out, expect, dtype, case["id"])
    if not training:
        return
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    out.features.backward(expect["grad_out"][inv].to(device).to(out.features.dtype))
    assert_close(feats.grad, expect["grad_input"], expect["atol_grad_input"], f"{case['id']}: grad_input")
    named = {f"{li}.{n}": p for li, layer in enumerate(layers) for n, p in layer.named_parameters()}
    assert set(named) == set(expect["grad_params"]), case["id"]
    for key, g in expect["grad_params"].items():
        assert_close(named[key].grad, g["grad"], g["atol"], f"{case['id']}: {key}.grad")


def build_unet3d(sp, in_channels=6, base=16):
    """The small UNet of the reference's network-level golden: submanifold stem
    with a shared key, strided down-conv, inverse up-conv, JoinTable, 1x1 head."""
    nn = torch.nn

    class UNet3d(nn.Module):
        def __init__(self):
            super().__init__()
            self.stem = sp.SparseSequential(
                sp.SubMConv3d(in_channels, base, 3, padding=1, indice_key="s0", bias=False),
                nn.BatchNorm1d(base), nn.ReLU(),
                sp.SubMConv3d(base, base, 3, padding=1, indice_key="s0", bias=False))
            self.down = sp.SparseConv3d(base, base * 2, 3, stride=2, padding=1, indice_key="d0", bias=False)
            self.mid = sp.SparseSequential(
                sp.SubMConv3d(base * 2, base * 2, 3, padding=1, indice_key="s1", bias=False),
                nn.BatchNorm1d(base * 2), nn.ReLU())
            self.up = sp.SparseInverseConv3d(base * 2, base, 3, indice_key="d0", bias=False)
            self.join = sp.JoinTable()
            self.head = sp.SubMConv3d(base * 2, 8, 1, bias=True)

        def forward(self, x):
            a = self.stem(x)
            d = self.up(self.mid(self.down(a)))
            return self.head(self.join([d, a]))

    return UNet3d()


def run_net_case(sp, case, device):
    dtype = getattr(torch, case["dtype"])
    net = build_unet3d(sp).to(device)
    net.load_state_dict(case["state_dict"])
    if dtype == torch.float16:
        net = net.half()
    net.train()
    inp = case["input"]
    feats = inp["features"].to(device).clone().requires_grad_(True)
    x = sp.SparseConvTensor(feats, inp["indices"].to(device), list(inp["spatial_shape"]), int(inp["batch_size"]))
    out = net(x)
    expect = case["expect"]
    order = check_sparse_output(out, expect, dtype, case["id"])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    out.features.backward(expect["grad_out"][inv].to(device).to(out.features.dtype))
    assert_close(feats.grad, expect["grad_input"], expect["atol_grad_input"], f"{case['id']}: grad_input")
    named = dict(net.named_parameters())
    for key, g in expect["grad_params"].items():
        assert_close(named[key].grad, g["grad"], g["atol"], f"{case['id']}: {key}.grad")
