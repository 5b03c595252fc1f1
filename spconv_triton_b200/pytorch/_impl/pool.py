"""Sparse max / average pooling through the C ABI.

Same four entry points as the reference module
spconv_triton/pytorch/_impl/pool.py (:260, :291, :333, :367).
"""

from __future__ import annotations

import torch

from spconv_triton_b200 import _lib


def maxpool_forward(features, pair_fwd, n_out):
    kv = int(pair_fwd.shape[0])
    feats = features.contiguous()
    c = int(feats.shape[1])
    dev = feats.device
    with torch.cuda.device(dev):
        out = torch.empty((n_out, c), dtype=feats.dtype, device=dev)
        if n_out == 0 or c == 0:
            return out
        pf = pair_fwd if pair_fwd.is_contiguous() else pair_fwd.contiguous()
        _lib.check(_lib.load().spc_maxpool_forward(_lib.ptr(feats), _lib.ptr(pf), _lib.ptr(out), n_out, c, kv,
                                                   _lib.dtype_code(feats.dtype), _lib.current_stream(dev)))
    return out


def maxpool_backward(features, out_features, grad_out, pair_bwd):
    kv = int(pair_bwd.shape[0])
    feats = features.contiguous()
    out = out_features.contiguous()
    g = grad_out.contiguous()
    n_in, c = feats.shape
    dev = feats.device
    with torch.cuda.device(dev):
        din = torch.zeros_like(feats)
        if n_in == 0 or c == 0:
            return din
        if g.dtype != feats.dtype:
            g = g.to(feats.dtype)
        pb = pair_bwd if pair_bwd.is_contiguous() else pair_bwd.contiguous()
        _lib.check(_lib.load().spc_maxpool_backward(_lib.ptr(feats), _lib.ptr(out), _lib.ptr(g), _lib.ptr(pb),
                                                    _lib.ptr(din), n_in, c, kv, _lib.dtype_code(feats.dtype),
                                                    _lib.current_stream(dev)))
    return din


def avgpool_forward(features, pair_fwd, n_out, calc_count=True):
    kv = int(pair_fwd.shape[0])
    feats = features.contiguous()
    c = int(feats.shape[1])
    dev = feats.device
    with torch.cuda.device(dev):
        out = torch.empty((n_out, c), dtype=feats.dtype, device=dev)
        count = torch.zeros((n_out,), dtype=torch.int32, device=dev)
        if n_out == 0 or c == 0:
            return out, count
        pf = pair_fwd if pair_fwd.is_contiguous() else pair_fwd.contiguous()
        _lib.check(_lib.load().spc_avgpool_forward(_lib.ptr(feats), _lib.ptr(pf), _lib.ptr(out),
                                                   _lib.ptr(count), n_out, c, kv,
                                                   _lib.dtype_code(feats.dtype), _lib.current_stream(dev)))
    return out, count


def avgpool_backward(grad_out, pair_bwd, count):
    kv = int(pair_bwd.shape[0])
    g = grad_out.contiguous()
    n_in = int(pair_bwd.shape[1])
    c = int(g.shape[1])
    dev = g.device
    with torch.cuda.device(dev):
        din = torch.zeros((n_in, c), dtype=g.dtype, device=dev)
        if n_in == 0 or c == 0:
            return din
        pb = pair_bwd if pair_bwd.is_contiguous() else pair_bwd.contiguous()
        cnt = count if count.is_contiguous() else count.contiguous()
        _lib.check(_lib.load().spc_avgpool_backward(_lib.ptr(g), _lib.ptr(pb), _lib.ptr(cnt), _lib.ptr(din),
                                                    n_in, c, kv, _lib.dtype_code(g.dtype),
                                                    _lib.current_stream(dev)))
    return din
