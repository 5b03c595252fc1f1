"""CPU oracle: gather-GEMM (forward, input gradient, weight gradient) and
sparse max/avg pooling over rulebook tables, restated with torch CPU tensors.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Formulas and the reference lines they follow:

* forward  out[m,n] = sum_k sum_c f[pf[k,m],c] * W[n,k,c] (+bias)
                                      spconv_triton/pytorch/_impl/gemm.py:254-258,313-315
* dgrad    din[j,c] = sum_k sum_n g[pb[k,j],n] * W[n,k,c]
                                      spconv_triton/pytorch/_impl/gemm.py:580-586
* wgrad    dW[n,k,c] = sum_{(i,o) in pairs_k} f[i,c] * g[o,n]
                                      spconv_triton/pytorch/_impl/gemm.py:356-369
* max pool (accumulator starts at 0), its backward (every tying input
  receives the gradient)              spconv_triton/pytorch/_impl/pool.py:75-86,148-149
* avg pool (divide by present count, >=1) and its backward (MULTIPLIES by the
  count)                              spconv_triton/pytorch/_impl/pool.py:200-201,250-252

All contractions are evaluated in ``acc_dtype`` (float64 by default) and the
result is rounded once to the requested output dtype, so the oracle is at
least as accurate as any accumulation order the reference's autotuner picks.
"""

from __future__ import annotations

import torch


def _as_long(t):
    return torch.as_tensor(t).long()


def _gather_rows(x, idx):
    """x[idx] with rows of zeros where idx < 0.  x: [n, c]; idx: [m] long."""
    safe = idx.clamp(min=0)
    rows = x.index_select(0, safe)
    return rows * (idx >= 0).unsqueeze(1).to(rows.dtype)


def conv_forward(features, w_krsc, pair_fwd, n_out, bias=None, out_dtype=None,
                 acc_dtype=torch.float64):
    """features [N,C]; w_krsc [K,kv,C]; pair_fwd [kv,n_out] -> [n_out,K]."""
    out_dtype = out_dtype or features.dtype
    pf = _as_long(pair_fwd)
    f = features.to(acc_dtype)
    w = w_krsc.to(acc_dtype)
    k_out, kv, _ = w.shape
    out = torch.zeros((n_out, k_out), dtype=acc_dtype)
    for k in range(kv):
        col = pf[k]
        if bool((col >= 0).any()):
            out += _gather_rows(f, col) @ w[:, k, :].t()
    if bias is not None:
        out += bias.to(acc_dtype)[None, :]
    return out.to(out_dtype)


def conv_backward_input(grad_out, w_krsc, pair_bwd, n_in, acc_dtype=torch.float64):
    """grad_out [M,K]; pair_bwd [kv,n_in] -> din [n_in,C] in grad_out.dtype."""
    pb = _as_long(pair_bwd)
    g = grad_out.to(acc_dtype)
    w = w_krsc.to(acc_dtype)
    _, kv, c_in = w.shape
    din = torch.zeros((n_in, c_in), dtype=acc_dtype)
    for k in range(kv):
        col = pb[k]
        if bool((col >= 0).any()):
            din += _gather_rows(g, col) @ w[:, k, :]
    return din.to(grad_out.dtype)


def conv_backward_weight(features, grad_out, pair_fwd, w_shape_krsc, acc_dtype=torch.float64):
    """-> dW [K,kv,C] in grad_out.dtype."""
    k_out, kv, c_in = w_shape_krsc
    pf = _as_long(pair_fwd)
    f = features.to(acc_dtype)
    g = grad_out.to(acc_dtype)
    dw = torch.zeros((k_out, kv, c_in), dtype=acc_dtype)
    for k in range(kv):
        col = pf[k]
        o = torch.nonzero(col >= 0, as_tuple=True)[0]
        if o.numel():
            dw[:, k, :] = g.index_select(0, o).t() @ f.index_select(0, col[o])
    return dw.to(grad_out.dtype)


def _acc_dtype_for(t):
    # pool.py:72-74: fp64 features keep an fp64 accumulator, everything else fp32.
    return torch.float64 if t.dtype == torch.float64 else torch.float32


def maxpool_forward(features, pair_fwd, n_out):
    pf = _as_long(pair_fwd)
    acc_t = _acc_dtype_for(features)
    f = features.to(acc_t)
    acc = torch.zeros((n_out, f.shape[1]), dtype=acc_t)
    neg = torch.full((1, f.shape[1]), float("-inf"), dtype=acc_t)
    for k in range(pf.shape[0]):
        col = pf[k]
        v = torch.where((col >= 0).unsqueeze(1), f.index_select(0, col.clamp(min=0)), neg)
        acc = torch.maximum(acc, v)
    return acc.to(features.dtype)


def maxpool_backward(features, out_features, grad_out, pair_bwd):
    pb = _as_long(pair_bwd)
    acc_t = _acc_dtype_for(features)
    n_in, c = features.shape
    acc = torch.zeros((n_in, c), dtype=acc_t)
    for k in range(pb.shape[0]):
        col = pb[k]
        ok = (col >= 0).unsqueeze(1)
        safe = col.clamp(min=0)
        o = out_features.index_select(0, safe)
        g = grad_out.index_select(0, safe).to(acc_t)
        hit = ok & (o == features)
        acc += torch.where(hit, g, torch.zeros_like(g))
    return acc.to(features.dtype)


def avgpool_forward(features, pair_fwd, n_out):
    """-> (out [n_out,C], count [n_out] int32)."""
    pf = _as_long(pair_fwd)
    acc_t = _acc_dtype_for(features)
    f = features.to(acc_t)
    acc = torch.zeros((n_out, f.shape[1]), dtype=acc_t)
    cnt = torch.zeros((n_out,), dtype=torch.int32)
    for k in range(pf.shape[0]):
        col = pf[k]
        acc += _gather_rows(f, col)
        cnt += (col >= 0).to(torch.int32)
    acc = acc / cnt.clamp(min=1).to(acc_t).unsqueeze(1)
    return acc.to(features.dtype), cnt


def avgpool_backward(grad_out, pair_bwd, count):
    pb = _as_long(pair_bwd)
    acc_t = _acc_dtype_for(grad_out)
    g = grad_out.to(acc_t)
    n_in = pb.shape[1]
    acc = torch.zeros((n_in, g.shape[1]), dtype=acc_t)
    cnt = torch.as_tensor(count).to(acc_t)
    for k in range(pb.shape[0]):
        col = pb[k]
        safe = col.clamp(min=0)
        contrib = g.index_select(0, safe) * cnt.index_select(0, safe).unsqueeze(1)
        acc += contrib * (col >= 0).unsqueeze(1).to(acc_t)
    return acc.to(grad_out.dtype)
