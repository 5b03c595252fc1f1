"""Generate tests/golden/ref_add.pt: golden vectors of the hash table and the misaligned sparse add.

Run once where the reference checkout is readable at $SPCONV_REFERENCE_ROOT:

    python tests/golden/make_golden_add.py

Four kinds of cases are written:
1. ``frozen``: the three ``sparse_add`` cases of the reference's own tests/data/golden_misc.pt
   (sparse_add, sparse_add_hash_based, add_table_misaligned), re-saved unchanged;
2. ``add``: outputs of the reference's ``functional.sparse_add_hash_based`` itself (pure torch,
   run here on the CPU) on seeded operands: three operands, full overlap, no overlap, an empty
   operand, 2-D, and a volume whose linear index needs int64;
3. ``table``: traces of the reference's ``hash.HashTable`` (CPU): repeated inserts with duplicate
   keys, query of absent keys, insert_exist_keys, assign_arange_, items with and without a limit.

Nothing here is imported by the product or by the tests.
"""

import importlib.metadata as _md
import os
import sys
from pathlib import Path

import torch

REF = os.environ["SPCONV_REFERENCE_ROOT"]  # the read-only reference checkout
OUT = Path(__file__).parent / "ref_add.pt"

_orig_version = _md.version
_md.version = lambda n: "1.0.0" if n == "spconv-triton" else _orig_version(n)
sys.path.insert(0, REF)

from spconv_triton.pytorch import functional as ref_f  # noqa: E402
from spconv_triton.pytorch.core import SparseConvTensor as RefTensor  # noqa: E402
from spconv_triton.pytorch.hash import HashTable as RefTable  # noqa: E402


def operand(g, shape, batch, channels, n, dtype=torch.float32):
    """n distinct voxels drawn from batch x shape, in random order."""
    total = batch
    for s in shape:
        total *= s
    if total <= 1 << 24:
        lin = torch.randperm(total, generator=g)[:n]
    else:
        lin = torch.unique(torch.randint(0, total, (2 * n + 8,), generator=g))
        lin = lin[torch.randperm(lin.numel(), generator=g)][:n]
    cols = []
    for s in reversed(shape):
        cols.append(lin % s)
        lin = lin // s
    cols.append(lin)
    idx = torch.stack(list(reversed(cols)), 1).int()
    feats = torch.randn(idx.shape[0], channels, generator=g).to(dtype)
    return dict(features=feats, indices=idx, spatial_shape=list(shape), batch_size=batch)


def run_add(inputs):
    tens = [RefTensor(i["features"].clone(), i["indices"].clone(), i["spatial_shape"], i["batch_size"]) for i in inputs]
    out = ref_f.sparse_add_hash_based(*tens)
    return dict(out_indices=out.indices, out_features=out.features, out_spatial_shape=list(out.spatial_shape))


def run_table(key_dtype, value_dtype, max_size, ops):
    """ops: list of (name, args...); returns the list of each op's result."""
    t = RefTable(torch.device("cpu"), key_dtype, value_dtype, max_size)
    res = []
    for op in ops:
        name, args = op[0], op[1:]
        r = getattr(t, name)(*[a.clone() if isinstance(a, torch.Tensor) else a for a in args])
        res.append(r)
    return res


def main():
    frozen = [c for c in torch.load(Path(REF) / "tests" / "data" / "golden_misc.pt", map_location="cpu",
                                    weights_only=False)["cases"] if c.get("kind") == "sparse_add"]
    g = torch.Generator().manual_seed(20240611)
    add = []

    def case(name, inputs):
        add.append(dict(id=name, inputs=inputs, expect=run_add(inputs)))

    a = operand(g, [24, 20, 16], 2, 16, 900)
    b = operand(g, [24, 20, 16], 2, 16, 700)
    c = operand(g, [24, 20, 16], 2, 16, 1100)
    case("three_operands", [a, b, c])
    same = dict(a, features=torch.randn(900, 16, generator=g))
    case("same_voxels", [a, same])
    perm = torch.randperm(900, generator=g)
    case("same_voxels_permuted", [a, dict(features=same["features"][perm], indices=a["indices"][perm],
                                          spatial_shape=a["spatial_shape"], batch_size=2)])
    lo = operand(g, [8, 8, 8], 1, 4, 100)
    hi = dict(lo, indices=lo["indices"] + torch.tensor([0, 8, 0, 0], dtype=torch.int32))
    lo16 = dict(lo, spatial_shape=[16, 8, 8])
    hi16 = dict(hi, spatial_shape=[16, 8, 8], features=torch.randn(100, 4, generator=g))
    case("disjoint", [lo16, hi16])
    empty = dict(features=torch.zeros(0, 16), indices=torch.zeros(0, 4, dtype=torch.int32),
                 spatial_shape=[24, 20, 16], batch_size=2)
    case("empty_operand", [a, empty])
    case("two_d_c3", [operand(g, [64, 48], 3, 3, 500), operand(g, [64, 48], 3, 3, 800)])
    case("half", [operand(g, [24, 20, 16], 2, 8, 600, torch.float16), operand(g, [24, 20, 16], 2, 8, 650, torch.float16)])
    case("int64_keys", [operand(g, [2000, 1500, 1200], 2, 4, 400), operand(g, [2000, 1500, 1200], 2, 4, 300)])

    tables = []

    def trace(name, key_dtype, value_dtype, max_size, ops):
        tables.append(dict(id=name, key_dtype=key_dtype, value_dtype=value_dtype, max_size=max_size, ops=ops,
                           expect=run_table(key_dtype, value_dtype, max_size, ops)))

    k1 = torch.randint(-500, 500, (300,), generator=g).int()        # many duplicates
    v1 = torch.randint(0, 1 << 20, (300,), generator=g).int()
    k2 = torch.randint(-500, 500, (200,), generator=g).int()
    v2 = torch.randint(0, 1 << 20, (200,), generator=g).int()
    q = torch.randint(-600, 600, (400,), generator=g).int()
    trace("int32_dups", torch.int32, torch.int32, 2048, [
        ("insert", k1, v1), ("query", q), ("insert", k2, v2), ("query", q), ("insert_exist_keys", q[:100], v1[:100]),
        ("query", q), ("items",), ("items", 50), ("assign_arange_",), ("query", q), ("items",)])
    k64 = torch.randint(-(1 << 50), 1 << 50, (500,), generator=g)
    k64[100:200] = k64[:100]
    v64 = torch.randn(500, generator=g)
    trace("int64_float", torch.int64, torch.float32, 1024, [
        ("insert", k64, v64), ("query", torch.cat([k64[:50], k64[:50] + 1])), ("items",), ("assign_arange_",),
        ("items",)])
    trace("no_values", torch.int32, torch.int64, 64, [
        ("insert", torch.tensor([9, 3, 3, 7], dtype=torch.int32)), ("query", torch.tensor([3, 4, 9], dtype=torch.int32)),
        ("assign_arange_",), ("query", torch.tensor([3, 7, 9, 1], dtype=torch.int32)), ("items",)])
    trace("empty_table", torch.int32, torch.int32, 16, [
        ("query", torch.tensor([1, 2], dtype=torch.int32)), ("assign_arange_",), ("items",),
        ("insert_exist_keys", torch.tensor([1], dtype=torch.int32), torch.tensor([5], dtype=torch.int32))])

    misc = torch.load(Path(REF) / "tests" / "data" / "golden_misc.pt", map_location="cpu", weights_only=False)["cases"]
    from_dense = [dict(id=c["id"], dense=c["dense"], indices=c["expect"]["indices"], features=c["expect"]["features"])
                  for c in misc if c.get("kind") == "from_dense"]
    torch.save(dict(frozen=frozen, add=add, table=tables, from_dense=from_dense), OUT)
    print("frozen", [c["id"] for c in frozen], "add", [c["id"] for c in add], "table", [t["id"] for t in tables])
    print(OUT, OUT.stat().st_size)


if __name__ == "__main__":
    main()
