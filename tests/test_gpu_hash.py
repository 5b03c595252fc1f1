"""CUDA hash table and misaligned sparse add (through the C ABI) against the reference's vectors
(tests/golden/ref_add.pt) and, on larger seeded inputs, against the numpy oracle."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import hash as oh

GOLD = torch.load(Path(__file__).parent / "golden" / "ref_add.pt", weights_only=False)
_NP = {torch.int32: np.int32, torch.int64: np.int64, torch.float32: np.float32}


def test_cpu_table_is_refused():
    from spconv_triton_b200.pytorch.hash import HashTable

    with pytest.raises(NotImplementedError):
        HashTable(torch.device("cpu"), torch.int32, torch.int32, 16)
    with pytest.raises(AssertionError):
        HashTable(torch.device("cuda"), torch.int32, torch.int32)      # CUDA tables need max_size
    with pytest.raises(AssertionError):
        HashTable(torch.device("cuda"), torch.float32, torch.int32, 16)


def tensors(case, fn="sparse_add_hash_based"):
    import spconv_triton_b200.pytorch as sp

    return [sp.SparseConvTensor(i["features"].cuda(), i["indices"].cuda(), i["spatial_shape"], i["batch_size"])
            for i in case["inputs"]]


def canonical(indices, features):
    key = torch.zeros(indices.shape[0], dtype=torch.int64)
    for d in range(indices.shape[1]):
        key = key * 100003 + indices[:, d]
    order = torch.argsort(key, stable=True)
    return indices[order], features[order]


@pytest.mark.gpu
@pytest.mark.parametrize("case", GOLD["frozen"], ids=lambda c: c["id"])
def test_frozen_sparse_add(case):
    import spconv_triton_b200.pytorch as sp

    tens = tensors(case)
    if case["fn"] == "add_table_misaligned":
        out = sp.AddTableMisaligned()(tens)
    else:
        out = getattr(sp.functional, case["fn"])(*tens)
    idx, feats = canonical(out.indices.cpu(), out.features.cpu())
    assert out.spatial_shape == case["expect"]["out_spatial_shape"]
    assert torch.equal(idx, case["expect"]["out_indices"])
    torch.testing.assert_close(feats, case["expect"]["out_features"], rtol=0, atol=case["expect"]["atol_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("case", GOLD["add"], ids=lambda c: c["id"])
def test_generated_sparse_add(case):
    import spconv_triton_b200.pytorch as sp

    out = sp.functional.sparse_add_hash_based(*tensors(case))
    assert torch.equal(out.indices.cpu(), case["expect"]["out_indices"])      # the reference's row order
    assert torch.equal(out.features.cpu(), case["expect"]["out_features"])    # bit-exact sums
    assert out.indices.dtype == torch.int32


@pytest.mark.gpu
@pytest.mark.parametrize("case", GOLD["table"], ids=lambda c: c["id"])
def test_table_trace(case):
    from spconv_triton_b200.pytorch.hash import HashTable

    table = HashTable(torch.device("cuda"), case["key_dtype"], case["value_dtype"], case["max_size"])
    for op, want in zip(case["ops"], case["expect"]):
        got = getattr(table, op[0])(*[a.cuda() if isinstance(a, torch.Tensor) else a for a in op[1:]])
        if op[0] == "insert":
            continue
        if op[0] == "assign_arange_":
            assert got.dtype == want.dtype and got.shape == want.shape and got.cpu().item() == want.item()
        elif op[0] == "insert_exist_keys":
            assert torch.equal(got.cpu(), want)
        else:
            for g, w in zip(got, want):
                assert g.dtype == w.dtype and torch.equal(g.cpu(), w), op[0]


@pytest.mark.gpu
def test_table_full_and_query_into():
    from spconv_triton_b200.pytorch.hash import HashTable

    table = HashTable(torch.device("cuda"), torch.int32, torch.int32, 4)
    table.insert(torch.arange(4, dtype=torch.int32), torch.arange(4, dtype=torch.int32) + 10)
    buf = torch.full((6,), -1, dtype=torch.int32, device="cuda")
    table.query(torch.tensor([2, 9], dtype=torch.int32), buf)
    assert buf.cpu().tolist() == [12, 0, -1, -1, -1, -1]
    with pytest.raises(AssertionError, match="hash table full"):
        table.insert(torch.arange(100, 140, dtype=torch.int32))


def big_operand(g, shape, batch, channels, n, dtype):
    total = batch * int(np.prod(shape))
    lin = torch.unique(torch.randint(0, total, (n,), generator=g))
    lin = lin[torch.randperm(lin.numel(), generator=g)]
    cols = []
    for s in reversed(shape):
        cols.append(lin % s)
        lin = lin // s
    cols.append(lin)
    idx = torch.stack(list(reversed(cols)), 1).int()
    return torch.randn(idx.shape[0], channels, generator=g).to(dtype), idx


@pytest.mark.gpu
@pytest.mark.parametrize("shape,channels,dtype", [([41, 400, 352], 64, torch.float16), ([41, 400, 352], 33, torch.float32),
                                                  ([1600, 1408, 1000], 16, torch.bfloat16)])
def test_large_against_oracle(shape, channels, dtype):
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(77)
    ops = [big_operand(g, shape, 2, channels, n, dtype) for n in (300_000, 250_000)]
    tens = [sp.SparseConvTensor(f.cuda(), i.cuda(), shape, 2) for f, i in ops]
    out = sp.functional.sparse_add(*tens)
    as_np = (lambda f: f.float().numpy()) if dtype == torch.bfloat16 else (lambda f: f.numpy())
    want_f, want_i = oh.sparse_add_hash_based([(as_np(f), i.numpy()) for f, i in ops], 2, shape)
    assert torch.equal(out.indices.cpu(), torch.from_numpy(want_i))
    want = torch.from_numpy(want_f).to(dtype)       # one addition per row: exact in fp32, rounded once
    assert torch.equal(out.features.cpu(), want)


@pytest.mark.gpu
def test_gradient_is_a_gather():
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(5)
    ops = [big_operand(g, [16, 16, 16], 2, 8, n, torch.float32) for n in (3000, 2500, 10)]
    feats = [f.cuda().requires_grad_(True) for f, _ in ops]
    tens = [sp.SparseConvTensor(f, i.cuda(), [16, 16, 16], 2) for f, (_, i) in zip(feats, ops)]
    out = sp.functional.sparse_add_hash_based(*tens)
    weight = torch.randn(out.features.shape, generator=g).cuda()
    (out.features * weight).sum().backward()
    lin_out = oh.indice_to_scalar(out.indices.cpu().numpy(), [2, 16, 16, 16])
    for f, (_, i) in zip(feats, ops):
        rows = np.searchsorted(lin_out, oh.indice_to_scalar(i.numpy(), [2, 16, 16, 16]))
        assert torch.equal(f.grad.cpu(), weight.cpu()[torch.from_numpy(rows)])


@pytest.mark.gpu
def test_indice_dict_follows_the_largest_operand():
    import spconv_triton_b200.pytorch as sp

    g = torch.Generator().manual_seed(9)
    f, i = big_operand(g, [16, 16, 16], 1, 4, 2000, torch.float32)
    a = sp.SparseConvTensor(f.cuda(), i.cuda(), [16, 16, 16], 1)
    a.indice_dict["k"] = "marker"
    b = sp.SparseConvTensor(f[:100].cuda(), i[:100].cuda(), [16, 16, 16], 1)
    assert sp.functional.sparse_add_hash_based(b, a).indice_dict.get("k") == "marker"
    with pytest.raises(AssertionError):
        sp.functional.sparse_add_hash_based(a, sp.SparseConvTensor(f.cuda(), i.cuda(), [16, 16, 8], 1))
