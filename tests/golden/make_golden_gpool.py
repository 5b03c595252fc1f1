"""Generate tests/golden/ref_gpool.pt: golden vectors of the global max / average pooling modules.

Run once where the reference checkout is readable at $SPCONV_REFERENCE_ROOT:

    python tests/golden/make_golden_gpool.py

Each case holds seeded features and indices, the output of the reference's SparseGlobalMaxPool /
SparseGlobalAvgPool (pure torch, run here on the CPU) and the gradient of sum(out * weight) with
respect to the features.  Values are distinct within a channel so that the maximum is unique.

Nothing here is imported by the product or by the tests.
"""

import importlib.metadata as _md
import os
import sys
from pathlib import Path

import torch

REF = os.environ["SPCONV_REFERENCE_ROOT"]  # the read-only reference checkout
OUT = Path(__file__).parent / "ref_gpool.pt"

_orig_version = _md.version
_md.version = lambda n: "1.0.0" if n == "spconv-triton" else _orig_version(n)
sys.path.insert(0, REF)

import spconv_triton.pytorch as ref_sp  # noqa: E402


def make(g, n, c, batch, dtype, order):
    # distinct values per channel: a permutation of an arithmetic grid, scaled into the dtype's exact range
    vals = torch.stack([torch.randperm(n, generator=g) for _ in range(c)], 1).float()
    feats = ((vals - n / 2) / 8).to(dtype)
    b = torch.randint(0, batch, (n,), generator=g)
    b[:batch] = torch.arange(batch)          # no empty sample
    if order == "sorted":
        b = torch.sort(b).values
    idx = torch.cat([b[:, None], torch.randint(0, 64, (n, 3), generator=g)], 1).int()
    return feats, idx


def run(feats, idx, batch, is_mean, weight):
    f = feats.float().clone().requires_grad_(True)   # the CPU run is in fp32 on the dtype's exact values
    x = ref_sp.SparseConvTensor(f, idx, [64, 64, 64], batch)
    mod = ref_sp.SparseGlobalAvgPool() if is_mean else ref_sp.SparseGlobalMaxPool()
    out = mod(x)
    (out * weight).sum().backward()
    return out.detach(), f.grad


def main():
    g = torch.Generator().manual_seed(20240613)
    cases = []
    for name, n, c, batch, dtype, order in [
            ("f32_shuffled", 1500, 16, 4, torch.float32, "shuffled"),
            ("f32_sorted_c130", 600, 130, 3, torch.float32, "sorted"),
            ("f16_sorted", 1024, 32, 8, torch.float16, "sorted"),
            ("bf16_shuffled", 200, 8, 2, torch.bfloat16, "shuffled"),
            ("one_row_per_sample", 5, 4, 5, torch.float32, "sorted")]:
        feats, idx = make(g, n, c, batch, dtype, order)
        for is_mean in (False, True):
            weight = torch.randn([batch] if is_mean else [batch, c], generator=g)
            out, grad = run(feats, idx, batch, is_mean, weight)
            cases.append(dict(id=f"{name}_{'mean' if is_mean else 'max'}", features=feats, indices=idx, batch_size=batch,
                              is_mean=is_mean, weight=weight, expect_out=out, expect_grad=grad))
    torch.save(dict(cases=cases), OUT)
    print([c["id"] for c in cases], OUT.stat().st_size)


if __name__ == "__main__":
    main()
