"""CPU restatement (numpy) of the reference's key -> value table and misaligned sparse add.

TEST INFRASTRUCTURE ONLY: nothing in the product imports this file.

Follows spconv_triton/pytorch/hash.py:15-110 (HashTable) and
spconv_triton/pytorch/functional.py:415-490 (_indice_to_scalar, sparse_add_hash_based).
Pinned by tests/test_oracle_hash.py against tests/golden/ref_add.pt, which holds the
reference's own frozen sparse_add cases and outputs of the reference run on the CPU.
"""

from __future__ import annotations

import numpy as np


class HashTable:
    """Sorted key array + value array, as hash.py:15-110 keeps them."""

    def __init__(self, key_dtype, value_dtype, max_size: int = -1):
        self.key_dtype = np.dtype(key_dtype)
        self.value_dtype = np.dtype(value_dtype)
        self.max_size = max_size
        self.keys = np.empty(0, self.key_dtype)
        self.values = np.empty(0, self.value_dtype)

    def insert(self, keys, values=None):  # hash.py:38-60
        keys = np.asarray(keys).astype(self.key_dtype).reshape(-1)
        values = (np.zeros(keys.shape[0], self.value_dtype) if values is None
                  else np.asarray(values).astype(self.value_dtype).reshape(-1))
        all_keys = np.concatenate([self.keys, keys])
        all_vals = np.concatenate([self.values, values])
        order = np.argsort(all_keys, kind="stable")
        sk, sv = all_keys[order], all_vals[order]
        last = np.ones(sk.shape[0], bool)
        last[:-1] = sk[1:] != sk[:-1]          # the last of equal keys wins
        self.keys, self.values = sk[last], sv[last]
        if self.max_size > 0 and self.keys.shape[0] > self.max_size:
            raise AssertionError("hash table full")

    def _find(self, keys):
        keys = np.asarray(keys).astype(self.key_dtype).reshape(-1)
        n = self.keys.shape[0]
        if n == 0:
            return keys, np.zeros(keys.shape[0], np.int64), np.zeros(keys.shape[0], bool)
        pos = np.searchsorted(self.keys, keys)
        pos_c = np.minimum(pos, n - 1)
        return keys, pos_c, (self.keys[pos_c] == keys) & (pos < n)

    def query(self, keys):  # hash.py:62-79
        keys, pos, found = self._find(keys)
        out = np.zeros(keys.shape[0], self.value_dtype)
        out[found] = self.values[pos[found]]
        return out, ~found

    def insert_exist_keys(self, keys, values):  # hash.py:81-92
        keys, pos, found = self._find(keys)
        values = np.asarray(values).astype(self.value_dtype).reshape(-1)
        self.values[pos[found]] = values[: keys.shape[0]][found]
        return found

    def assign_arange_(self):  # hash.py:94-99
        self.values = np.arange(self.keys.shape[0]).astype(self.value_dtype)
        return self.keys.shape[0]

    def items(self, max_size: int = -1):  # hash.py:101-110
        if max_size == -1:
            max_size = self.max_size
        n = min(self.keys.shape[0], max_size)
        k = np.zeros(max_size, self.key_dtype)
        v = np.zeros(max_size, self.value_dtype)
        k[:n], v[:n] = self.keys[:n], self.values[:n]
        return k, v, n


def indice_to_scalar(indices, shape):  # functional.py:415-426
    lin = np.zeros(indices.shape[0], np.int64)
    for d, s in enumerate(shape):
        lin = lin * int(s) + indices[:, d].astype(np.int64)
    return lin


def sparse_add_hash_based(operands, batch_size, spatial_shape):
    shape = [batch_size, *spatial_shape]
    table = HashTable(np.int64, np.int32, -1)
    scalars = [indice_to_scalar(idx, shape) for _, idx in operands]
    for s in scalars:
        table.insert(s)
    count = table.assign_arange_()
    feats0, idx0 = operands[0]
    out_f = np.zeros((count, feats0.shape[1]), feats0.dtype)
    out_i = np.zeros((count, idx0.shape[1]), idx0.dtype)
    for (f, idx), s in zip(operands, scalars):
        rows, _ = table.query(s)
        out_f[rows] = out_f[rows] + f          # rows are distinct within one operand
        out_i[rows] = idx
    return out_f, out_i
