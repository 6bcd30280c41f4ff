"""The C-ABI library loads and exports every symbol include/leviathan_cuda.h
declares (no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

import pytest

from leviathan_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "leviathan_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lev_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(L.LIB_PATH):
        from leviathan_b200.build import build_library

        build_library()
    return ctypes.CDLL(L.LIB_PATH)


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared but not exported"


def test_binding_table_matches_header():
    assert sorted(L.SIGNATURES) == _declared_symbols()


def test_version_and_status_names(lib):
    lib.lev_cuda_abi_version.restype = ctypes.c_int
    assert lib.lev_cuda_abi_version() == 1
    lib.lev_status_name.restype = ctypes.c_char_p
    for code, name in L.STATUS.items():
        assert lib.lev_status_name(code).decode() == name


def test_init_without_a_gpu_fails_with_a_status_not_a_crash(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    lib.lev_cuda_init.restype = ctypes.c_int
    st = lib.lev_cuda_init(0, ctypes.byref(h))
    assert st == 8 and not h.value  # LEV_DEVICE_UNAVAILABLE


def test_package_fails_loudly_when_library_is_missing(monkeypatch):
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", "/nonexistent/libleviathan_cuda.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        L.load()
