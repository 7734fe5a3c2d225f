"""The C-ABI library loads without a GPU and exports every symbol include/crownest_ops.h declares."""
import ctypes
import os
import re

from conftest import ROOT
from crownest_b200 import _lib


def header_symbols():
    text = open(os.path.join(ROOT, "include", "crownest_ops.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_lib.SO_PATH)
    names = header_symbols()
    assert len(names) >= 7
    for n in names:
        assert hasattr(L, n), f"{n} is declared in the header but not exported"
    # and the Python binding knows each of them
    assert set(names) <= set(_lib.exported_symbols()), set(names) - set(_lib.exported_symbols())


def test_error_string_and_version_need_no_gpu():
    L = _lib.lib()
    assert b"sm_100a" in L.cn_version()
    # a refused shape is reported before any CUDA call
    assert L.cn_nvfp4_gemv(None, None, None, None, 4, 100, 1, 4, 1, None) == 1
    assert b"multiple of 256" in L.cn_last_error_string()
