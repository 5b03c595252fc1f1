"""Helpers for users' unit tests, with the names of the reference's
spconv_triton/test_utils.py: a ``TestCase`` with array assertions, the
cartesian ``params_grid`` and the random voxel-data generator (which draws
from numpy's GLOBAL random state in the same order as upstream, so seeded
results agree)."""

from __future__ import annotations

import itertools
import unittest

import numpy as np


class TestCase(unittest.TestCase):
    def assertAllEqual(self, a, b):
        """Same shape and same values; NaNs at the same places count as equal."""
        a, b = np.asarray(a), np.asarray(b)
        self.assertEqual(a.shape, b.shape, f"Shape mismatch: expected {a.shape}, got {b.shape}.")
        np.testing.assert_array_equal(a, b)

    def assertAllClose(self, a, b, rtol=1e-6, atol=1e-6, msg: str = ""):
        """Arrays, or flat dicts of arrays with the same keys, equal within rtol / atol."""
        if isinstance(a, dict) != isinstance(b, dict):
            raise ValueError(f"Can't compare dict to non-dict, {a} vs {b}. {msg}")
        if isinstance(a, dict):
            self.assertCountEqual(a.keys(), b.keys(), msg=f"mismatched keys, expected {a.keys()}, got {b.keys()}. {msg}")
            for key in a:
                self.assertAllClose(a[key], b[key], rtol=rtol, atol=atol, msg=f"{key}: {msg}")
            return
        a, b = np.asarray(a), np.asarray(b)
        self.assertEqual(a.shape, b.shape, f"Shape mismatch: expected {a.shape}, got {b.shape}.")
        np.testing.assert_allclose(a, b, rtol=rtol, atol=atol, err_msg=msg)


def params_grid(*params):
    """Every combination of one element per list, last list varying fastest."""
    return [list(combo) for combo in itertools.product(*params)]


def generate_sparse_data(shape, num_points, num_channels, integer=False, data_range=(-1, 1), with_dense=True,
                         dtype=np.float32, shape_scale=1):
    """Random voxels for a batch: per sample ``num_points[b]`` distinct cells of the
    grid ``shape`` (on a lattice of stride ``shape_scale``) with ``num_channels``
    features.  Returns ``features`` [N, C], ``indices`` [N, ndim + 1] int32 with the
    batch index in the LAST column, and (``with_dense``) ``features_dense``
    [batch, C, *shape]."""
    ndim = len(shape)
    counts = np.array(num_points)
    cells = np.stack(np.meshgrid(*[np.arange(0, s // shape_scale) for s in shape]), axis=-1).reshape(-1, ndim)
    cells = cells * shape_scale
    per_sample = []
    for b in range(len(counts)):
        np.random.shuffle(cells)  # one shuffle per sample, as upstream: keeps seeded results identical
        per_sample.append(np.concatenate([cells[:counts[b]], np.full((counts[b], 1), b, cells.dtype)], axis=1))
    total = int(counts.sum())
    if integer:
        feats = np.random.randint(data_range[0], data_range[1], size=[total, num_channels]).astype(dtype)
    else:
        feats = np.random.uniform(data_range[0], data_range[1], size=[total, num_channels]).astype(dtype)
    out = {"features": feats}
    if with_dense:
        dense = np.zeros([len(counts), num_channels, *shape], dtype=feats.dtype)
        start = 0
        for b, rows in enumerate(per_sample):
            where = (b, slice(None)) + tuple(rows[:, d] for d in range(ndim))
            dense[where] = feats[start:start + len(rows)]
            start += len(rows)
        out["features_dense"] = dense
    out["indices"] = np.concatenate(per_sample, axis=0).astype(np.int32)
    return out
