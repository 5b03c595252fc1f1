"""Test-only adapter: lets the package's host-side layers (modules, autograd
functions, operator adaptors) run on CPU tensors by pointing the operator
layer at the CPU oracle instead of libspconv_b200.so.

Only tests use this (never the product): it checks the host logic and pins the
oracle against the reference's frozen network-level golden cases without a GPU.
"""

from types import SimpleNamespace

import numpy as np
import torch

from oracle import features as of
from oracle import rulebook as orb


def _t(a, dtype=torch.int32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype)


def _igemm_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                 transpose, is_train, is_mask_split, do_sort=True, num_out_act_bound=-1):
    res = orb.igemm_pairs(indices.numpy(), batch_size, spatial_shape, ksize, stride, padding, dilation,
                          out_padding, subm, transpose, is_train, is_mask_split, do_sort, num_out_act_bound)
    out_inds, npl, pf, pb, pmf, pmb, maf, mab, masks = res
    return (indices if subm else _t(out_inds), _t(npl), _t(pf), _t(pb) if pb is not None else torch.Tensor(),
            [_t(m) for m in pmf], [_t(m) for m in pmb], [_t(m) for m in maf], [_t(m) for m in mab], masks)


def _native_pairs(indices, batch_size, spatial_shape, ksize, stride, padding, dilation, out_padding, subm,
                  transpose):
    out_inds, pair, npl = orb.native_pairs(indices.numpy(), batch_size, spatial_shape, ksize, stride, padding,
                                           dilation, out_padding, subm, transpose)
    return (indices if subm else _t(out_inds)), _t(pair), _t(npl)


def _native_pair_to_tables(pair, indice_pair_num, n_in, n_out, inverse, need_bwd=True):
    pf, pb = orb.native_pair_to_tables(pair.numpy(), n_in, n_out, inverse, need_bwd)
    return _t(pf), (_t(pb) if pb is not None else None)


def _conv_forward(features, w, pair_fwd, n_out, bias=None, out_dtype=None, pair_mask=None, mask_argsort=None,
                  fp32_accum=None, epilogue=None, residual=None):
    scale, shift, act, alpha = epilogue if epilogue is not None else (None, None, 0, 0.0)
    out_dtype = out_dtype or features.dtype
    out = of.conv_forward(features.detach(), w.detach(), pair_fwd, n_out, bias=None if bias is None else bias.detach(),
                          out_dtype=torch.float64)
    if scale is not None:
        out = out * scale.double() + shift.double()
    if act == 1:
        out = torch.relu(out)
    elif act == 2:
        out = torch.sigmoid(out)
    elif act == 3:
        out = torch.nn.functional.leaky_relu(out, alpha)
    if residual is not None:
        out = out + residual.detach().double()
    return out.to(out_dtype)


def _conv_backward_input(grad_out, w, pair_bwd, n_in, pair_mask=None, mask_argsort=None, fp32_accum=None):
    return of.conv_backward_input(grad_out, w.detach(), pair_bwd, n_in)


def _conv_backward_weight(features, grad_out, pair_fwd, w_shape, fp32_accum=None):
    return of.conv_backward_weight(features.detach(), grad_out, pair_fwd, tuple(int(v) for v in w_shape))


def install(monkeypatch):
    """Point ``spconv_triton_b200.pytorch.ops`` at the oracle for one test."""
    from spconv_triton_b200.pytorch import ops

    monkeypatch.setattr(ops, "_pairs", SimpleNamespace(
        igemm_pairs=_igemm_pairs, native_pairs=_native_pairs, native_pair_to_tables=_native_pair_to_tables))
    monkeypatch.setattr(ops, "_gemm", SimpleNamespace(
        conv_forward=_conv_forward, conv_backward_input=_conv_backward_input,
        conv_backward_weight=_conv_backward_weight))
    monkeypatch.setattr(ops, "_pool", SimpleNamespace(
        maxpool_forward=lambda f, pf, n: of.maxpool_forward(f.detach(), pf, n),
        maxpool_backward=lambda f, o, g, pb: of.maxpool_backward(f.detach(), o.detach(), g, pb),
        avgpool_forward=lambda f, pf, n, calc_count=True: of.avgpool_forward(f.detach(), pf, n),
        avgpool_backward=lambda g, pb, c: of.avgpool_backward(g, pb, c)))
    monkeypatch.setattr(ops, "_require_cuda", lambda t, msg="": None)
