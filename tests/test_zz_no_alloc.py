"""The workspace-free weight-gradient entry point, called through the C ABI.

It exists for hosts that embed the library as a plugin and may neither allocate
device memory nor pass a workspace (see include/spconv_b200.h).  Its result must
equal that of the regular entry point, which gets its scratch from the caller --
also on a second call, when the built-in scratch still holds the first call's
partial sums.  Collected last on purpose (file name), so that a failure here
cannot hide failures elsewhere when pytest stops at the first one.
"""

import ctypes

import numpy as np
import pytest
import torch

from gpu_util import DEV, unique_coords
from oracle import features as of
from oracle import rulebook as orb

pytestmark = pytest.mark.gpu


def _tables(seed, n):
    shape, batch = [24, 40, 36], 2
    idx = unique_coords(seed, n, batch, shape)
    res = orb.igemm_pairs(idx, batch, shape, [3] * 3, [2] * 3, [1] * 3, [1] * 3, [0] * 3, False, False, True, False)
    return idx.shape[0], torch.from_numpy(res[2]).to(DEV)


def _both(lib, _lib, feats, gout, pf, c_in, c_out, dtype):
    kv, n_out = pf.shape
    stream = _lib.current_stream(feats.device)
    code = _lib.dtype_code(dtype)
    ref = torch.empty((c_out, kv, c_in), dtype=dtype, device=DEV)
    nbytes = int(lib.spc_conv_backward_weight_workspace_bytes(n_out, c_in, c_out, kv))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    _lib.check(lib.spc_conv_backward_weight(_lib.ptr(feats), _lib.ptr(gout), _lib.ptr(pf), _lib.ptr(ref), _lib.ptr(ws),
                                            nbytes, feats.shape[0], n_out, c_in, c_out, kv, code, _lib.SPC_PREC_IEEE,
                                            _lib.SPC_GEMM_SIMT, stream))
    got = torch.full((c_out, kv, c_in), float("nan"), dtype=dtype, device=DEV)
    _lib.check(lib.spc_conv_backward_weight_noalloc(_lib.ptr(feats), _lib.ptr(gout), _lib.ptr(pf), _lib.ptr(got),
                                                    feats.shape[0], n_out, c_in, c_out, kv, code, stream))
    torch.cuda.synchronize()
    return ref, got


def test_matches_regular_entry_point_on_two_calls_in_a_row():
    from spconv_triton_b200 import _lib

    lib = _lib.load()
    assert lib.spc_conv_backward_weight_noalloc_max_bytes() == 16 << 20
    gen = torch.Generator().manual_seed(3)
    # two different problems back to back: the second must not see the first one's partial sums
    for seed, n, c_in, c_out, dtype in ((21, 9000, 32, 48, torch.float16), (22, 5000, 16, 24, torch.float32)):
        n_in, pf = _tables(seed, n)
        feats = torch.randn(n_in, c_in, generator=gen).to(dtype).to(DEV)
        gout = torch.randn(pf.shape[1], c_out, generator=gen).to(dtype).to(DEV)
        ref, got = _both(lib, _lib, feats, gout, pf, c_in, c_out, dtype)
        # same kernels, same split, same summation order: identical bits
        assert torch.equal(ref, got)
        scale = ref.float().abs().max().item()
        assert np.isfinite(scale) and scale > 0
        # and the sum itself, against the fp64 oracle over the same table
        expect = of.conv_backward_weight(feats.cpu().double(), gout.cpu().double(), pf.cpu().numpy(),
                                         (c_out, pf.shape[0], c_in))
        err = (got.cpu().double() - expect).abs().max().item() / expect.abs().max().item()
        assert err <= (2e-3 if dtype == torch.float16 else 1e-5), f"{dtype}: {err:.2e}"


def test_rejects_shapes_beyond_the_built_in_scratch():
    from spconv_triton_b200 import _lib

    lib = _lib.load()
    c, kv, n_out = 512, 27, 1000  # 512 * 27 * 512 * 4 bytes = 27 MiB of partial sums > 16 MiB
    assert lib.spc_conv_backward_weight_workspace_bytes(n_out, c, c, kv) > lib.spc_conv_backward_weight_noalloc_max_bytes()
    feats = torch.zeros((8, c), dtype=torch.float16, device=DEV)
    gout = torch.zeros((n_out, c), dtype=torch.float16, device=DEV)
    pf = torch.full((kv, n_out), -1, dtype=torch.int32, device=DEV)
    dw = torch.empty((c, kv, c), dtype=torch.float16, device=DEV)
    rc = lib.spc_conv_backward_weight_noalloc(_lib.ptr(feats), _lib.ptr(gout), _lib.ptr(pf), _lib.ptr(dw), 8, n_out, c, c,
                                              kv, _lib.SPC_F16, _lib.current_stream(feats.device))
    assert rc == 7  # SPC_ERR_SIZE_LIMIT
    assert b"built-in scratch" in lib.spc_last_error()
