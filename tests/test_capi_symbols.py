"""The C-ABI library loads without a GPU and exports every function the
header declares; host-only entry points give the reference's known answers."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "spconv_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spc_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    from spconv_triton_b200 import _lib

    assert declared_functions() == sorted(set(_lib.exported_symbols()) | set(_lib._OPTIONAL))


def test_library_exports_every_declared_symbol():
    from spconv_triton_b200 import _lib

    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"libspconv_b200.so does not export {name}"
    assert lib.spc_version() >= 100


def test_output_size_known_answers():
    # the literals the reference pins (tests/test_ops.py:22-38 in the reference project)
    from spconv_triton_b200.pytorch import ops

    assert ops.get_conv_output_size([41, 1600, 1408], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1]) == [21, 800, 704]
    assert ops.get_conv_output_size([10], [-1], [1], [0], [1]) == [1]
    assert ops.get_conv_output_size([7, 9], [3, 2], [2, 1], [1, 0], [1, 1]) == [4, 8]
    assert ops.get_conv_output_size([2], [5], [1], [0], [1]) == [-2]
    assert ops.get_deconv_output_size([8, 8, 8], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1], [1, 1, 1]) == [16, 16, 16]
    with pytest.raises(ValueError):
        ops.get_deconv_output_size([8], [-1], [1], [0], [1], [0])


def test_workspace_query_needs_no_gpu():
    from spconv_triton_b200 import _lib

    g = _lib.make_geometry(4, [41, 1600, 1408], [21, 800, 704], [3, 3, 3], [2, 2, 2], [1, 1, 1], [1, 1, 1],
                           False, False)
    nbytes = _lib.load().spc_rulebook_workspace_bytes(ctypes.byref(g), 480000)
    assert 0 < nbytes < (1 << 31)
    assert _lib.load().spc_conv_backward_weight_workspace_bytes(100000, 64, 64, 27) > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from spconv_triton_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
