"""The C-ABI library on a machine without a GPU: it loads, exports every symbol that
include/alpha_cuda.h declares, and refuses to compute without a device."""
import ctypes
import os
import re

import pytest

from alpha2_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "alpha_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(alpha_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = _declared()
    assert len(names) > 70
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_covers_the_header():
    bound = set(L.exported_names())
    assert set(_declared()) <= bound, sorted(set(_declared()) - bound)


def test_no_compute_without_init():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = L.load()
    assert lib.alpha_init(0) != 0
    assert b"no CPU fallback" in lib.alpha_last_error()
    out = ctypes.c_uint64()
    assert lib.alpha_alloc(16, ctypes.byref(out)) != 0
    assert b"alpha_init was not called" in lib.alpha_last_error()
    assert lib.alpha_gemm(0, 0, 0, 0, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 0, 0) != 0


def test_missing_library_is_loud(monkeypatch, tmp_path):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "SO_PATH", str(tmp_path / "libalpha_cuda.so"))
    with pytest.raises(L.AlphaCudaError, match="no CPU or PyTorch fallback"):
        L.load()
