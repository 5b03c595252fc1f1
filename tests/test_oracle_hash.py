"""The numpy restatement of the hash table and the misaligned sparse add against the reference's
own vectors (tests/golden/ref_add.pt: frozen cases of the reference + reference outputs)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import hash as oh

GOLD = torch.load(Path(__file__).parent / "golden" / "ref_add.pt", weights_only=False)
_NP = {torch.int32: np.int32, torch.int64: np.int64, torch.float32: np.float32}


def canonical(indices, features):
    key = np.zeros(indices.shape[0], np.int64)
    for d in range(indices.shape[1]):
        key = key * 100003 + indices[:, d]
    order = np.argsort(key, kind="stable")
    return indices[order], features[order]


def run_oracle(case):
    ops = [(i["features"].numpy(), i["indices"].numpy()) for i in case["inputs"]]
    first = case["inputs"][0]
    return oh.sparse_add_hash_based(ops, first["batch_size"], first["spatial_shape"])


@pytest.mark.parametrize("case", GOLD["frozen"], ids=lambda c: c["id"])
def test_frozen_sparse_add(case):
    out_f, out_i = run_oracle(case)
    out_i, out_f = canonical(out_i, out_f)
    np.testing.assert_array_equal(out_i, case["expect"]["out_indices"].numpy())
    np.testing.assert_allclose(out_f, case["expect"]["out_features"].numpy(), rtol=0, atol=case["expect"]["atol_out"])


@pytest.mark.parametrize("case", GOLD["add"], ids=lambda c: c["id"])
def test_generated_sparse_add(case):
    out_f, out_i = run_oracle(case)
    np.testing.assert_array_equal(out_i, case["expect"]["out_indices"].numpy())       # same row order
    np.testing.assert_array_equal(out_f, case["expect"]["out_features"].numpy())      # bit-exact sums


def replay(table, ops):
    res = []
    for op in ops:
        name, args = op[0], [a.numpy() if isinstance(a, torch.Tensor) else a for a in op[1:]]
        res.append(getattr(table, name)(*args))
    return res


@pytest.mark.parametrize("case", GOLD["table"], ids=lambda c: c["id"])
def test_table_trace(case):
    table = oh.HashTable(_NP[case["key_dtype"]], _NP[case["value_dtype"]], case["max_size"])
    for op, got, want in zip(case["ops"], replay(table, case["ops"]), case["expect"]):
        if op[0] == "insert":
            continue
        if op[0] == "assign_arange_":
            assert got == int(want.item())
        elif op[0] == "insert_exist_keys":
            np.testing.assert_array_equal(got, want.numpy())
        elif op[0] == "query":
            np.testing.assert_array_equal(got[0], want[0].numpy())
            np.testing.assert_array_equal(got[1], want[1].numpy())
        else:
            np.testing.assert_array_equal(got[0], want[0].numpy())
            np.testing.assert_array_equal(got[1], want[1].numpy())
            assert got[2] == int(want[2].item())


def test_table_full():
    table = oh.HashTable(np.int32, np.int32, 4)
    with pytest.raises(AssertionError):
        table.insert(np.arange(5))
