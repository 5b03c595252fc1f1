"""CPU oracle: a whole sparse backbone evaluated with the oracle's rulebook,
gather-GEMM and pooling functions.

TEST INFRASTRUCTURE ONLY.  Used to check network-level outputs of the CUDA
path and, timed, as the CPU baseline of the benchmark.  The layer list is the
same plain description the benchmark builds its model from.
"""

from __future__ import annotations

import numpy as np
import torch

from . import features as of
from . import rulebook as orb


def run_backbone(layers, params, indices, features, spatial_shape, batch_size, acc_dtype=torch.float32,
                 stats=None):
    """``layers``: list of dicts {kind: subm|conv, cin, cout, k, s, p, key};
    every layer is followed by BatchNorm1d (inference statistics) and ReLU.
    ``params[i]``: dict(weight [K,kv,C], bn_weight, bn_bias, bn_mean, bn_var, eps).
    Returns (out_indices, out_features, out_spatial_shape)."""
    idx = np.asarray(indices)
    feats = features
    shape = list(spatial_shape)
    cache = {}
    for li, (L, P) in enumerate(zip(layers, params)):
        nd = len(shape)
        k, s, p = [L["k"]] * nd, [L["s"]] * nd, [L["p"]] * nd
        subm = L["kind"] == "subm"
        key = L.get("key")
        if subm and key in cache:
            pf = cache[key]
        else:
            res = orb.igemm_pairs(idx, batch_size, shape, k, s, p, [1] * nd, [0] * nd, subm, False,
                                  not subm, False)
            pf = res[2]
            if subm and key is not None:
                cache[key] = pf
            if not subm:
                idx = res[0]
                shape = orb.conv_output_size(shape, k, s, p, [1] * nd)
        n_out = pf.shape[1]
        if stats is not None:
            stats.append(dict(layer=li, n_out=int(n_out), pairs=int((pf >= 0).sum()), cin=L["cin"], cout=L["cout"]))
        y = of.conv_forward(feats, P["weight"], pf, n_out, acc_dtype=acc_dtype, out_dtype=feats.dtype)
        y = y.float()
        y = (y - P["bn_mean"]) / torch.sqrt(P["bn_var"] + P["eps"]) * P["bn_weight"] + P["bn_bias"]
        feats = torch.relu(y).to(features.dtype)
    return idx, feats, shape
