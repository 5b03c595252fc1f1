"""HashTable with the interface of the reference's
``spconv_triton/pytorch/hash.py:15-110`` on a CUDA open-addressing table.

The reference keeps two sorted arrays and re-sorts them on every insert; the
observable behaviour kept here is: a key inserted again takes the new value
(within one call the last occurrence wins), ``query`` returns 0 / is_empty for
absent keys, ``assign_arange_`` numbers the keys in ascending key order and
``items`` lists the pairs in that order.  All table work runs in
``libspconv_b200`` (``csrc/hash.cu``); there is no CPU table: a CPU device
raises NotImplementedError.
"""

from __future__ import annotations

import ctypes

import torch

from spconv_triton_b200 import _lib


def _pow2_at_least(n: int) -> int:
    p = 2
    while p < n:
        p *= 2
    return p


class HashTable:
    def __init__(self, device: torch.device, key_dtype: torch.dtype, value_dtype: torch.dtype, max_size: int = -1):
        device = torch.device(device)
        if key_dtype not in (torch.int32, torch.int64):
            raise AssertionError
        if device.type != "cpu" and max_size <= 0:
            raise AssertionError("you must provide max_size for fixed-size cuda hash table, "
                                 "usually *2 of num of keys")
        if device.type != "cuda":
            raise NotImplementedError("spconv_triton_b200.pytorch.hash.HashTable is CUDA only")
        if torch.empty(0, dtype=value_dtype).element_size() not in (1, 2, 4, 8):
            raise NotImplementedError(f"value dtype {value_dtype} is not supported")
        self.device = device
        self.key_dtype = key_dtype
        self.value_dtype = value_dtype
        self.max_size = int(max_size)
        self._lib = _lib.load()
        self._cap = _pow2_at_least(2 * self.max_size)
        self._buf = torch.empty(self._lib.spc_hash_bytes(self._cap), dtype=torch.uint8, device=device)
        self._epoch = 0
        self._key_bits = 0  # set by callers that know every key is in [0, 2^bits): shortens the sort
        self._call("spc_hash_clear", _lib.ptr(self._buf), self._cap)

    # -- plumbing ---------------------------------------------------------------------------
    def _call(self, name, *args):
        with torch.cuda.device(self.device):
            _lib.check(getattr(self._lib, name)(*args, _lib.current_stream(self.device)))

    def _keys(self, keys: torch.Tensor) -> torch.Tensor:
        return keys.to(self.device).to(self.key_dtype).reshape(-1).contiguous()

    def _values(self, values: torch.Tensor) -> torch.Tensor:
        return values.to(self.device).to(self.value_dtype).reshape(-1).contiguous()

    @property
    def _kb(self) -> int:
        return 4 if self.key_dtype == torch.int32 else 8

    @property
    def _vb(self) -> int:
        return torch.empty(0, dtype=self.value_dtype).element_size()

    def _counters(self) -> tuple[int, int]:
        stored, dropped = ctypes.c_int64(0), ctypes.c_int64(0)
        self._call("spc_hash_counters", _lib.ptr(self._buf), self._cap, ctypes.byref(stored), ctypes.byref(dropped))
        return stored.value, dropped.value

    # -- the reference's interface ----------------------------------------------------------
    def insert(self, keys: torch.Tensor, values: torch.Tensor | None = None):
        self._insert_unchecked(keys, values)
        stored, dropped = self._counters()
        if dropped > 0 or stored > self.max_size:
            raise AssertionError("hash table full")

    def _insert_unchecked(self, keys: torch.Tensor, values: torch.Tensor | None = None):
        """insert without the host read of the fill count (for callers that sized the table for all keys)."""
        keys = self._keys(keys)
        if values is not None:
            values = self._values(values)
            if values.shape[0] < keys.shape[0]:
                raise AssertionError("fewer values than keys")
        self._epoch += 1
        self._call("spc_hash_insert", _lib.ptr(self._buf), self._cap, _lib.ptr(keys), self._kb, _lib.ptr(values),
                   self._vb, int(keys.shape[0]), self._epoch)

    def query(self, keys: torch.Tensor, values: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        keys = self._keys(keys)
        n = int(keys.shape[0])
        out_v = torch.empty(n, dtype=self.value_dtype, device=self.device)
        is_empty = torch.empty(n, dtype=torch.bool, device=self.device)
        self._call("spc_hash_query", _lib.ptr(self._buf), self._cap, _lib.ptr(keys), self._kb, n, _lib.ptr(out_v),
                   self._vb, _lib.ptr(is_empty))
        if values is not None:
            values.reshape(-1)[:n].copy_(out_v)
        return out_v, is_empty

    def insert_exist_keys(self, keys: torch.Tensor, values: torch.Tensor):
        keys = self._keys(keys)
        values = self._values(values)
        n = int(keys.shape[0])
        if values.shape[0] < n:
            raise AssertionError("fewer values than keys")
        found = torch.empty(n, dtype=torch.bool, device=self.device)
        self._call("spc_hash_update", _lib.ptr(self._buf), self._cap, _lib.ptr(keys), self._kb, _lib.ptr(values),
                   self._vb, n, _lib.ptr(found))
        return found

    def _items(self, assign_kind: int, out_keys, out_values, limit: int) -> int:
        stored, _ = self._counters()
        if stored > 0:
            ws = torch.empty(self._lib.spc_hash_items_workspace_bytes(stored), dtype=torch.uint8, device=self.device)
            self._call("spc_hash_items", _lib.ptr(self._buf), self._cap, stored, assign_kind, self._key_bits,
                       _lib.ptr(ws), ws.numel(), _lib.ptr(out_keys), self._kb, _lib.ptr(out_values), self._vb,
                       int(limit))
        return stored

    def _count_tensor(self, n: int) -> torch.Tensor:
        count_dtype = torch.int32 if self.key_dtype == torch.int32 else torch.int64
        return torch.tensor([n], dtype=count_dtype, device=self.device)

    def assign_arange_(self):
        if self.value_dtype.is_floating_point:
            if self.value_dtype not in (torch.float32, torch.float64):
                raise NotImplementedError(f"assign_arange_ with {self.value_dtype} values")
            kind = 1 if self.value_dtype == torch.float32 else 2
        else:
            kind = 0
        return self._count_tensor(self._items(kind, None, None, 0))

    def items(self, max_size: int = -1):
        if max_size == -1:
            max_size = self.max_size
        keys = torch.zeros([max_size], dtype=self.key_dtype, device=self.device)
        values = torch.zeros([max_size], dtype=self.value_dtype, device=self.device)
        n = min(self._items(-1, keys, values, max_size), max_size)
        return keys, values, self._count_tensor(n)
