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


def test_shared_memory_attribute_is_booked_per_kernel_and_device():
    """The large dynamic shared-memory attribute belongs to a (kernel, device) pair: a process that launches on a second
    GPU must set it there again, and a larger request on the same GPU too. cn_smem_book is the book every launch consults."""
    L = _lib.lib()
    k1, k2 = ctypes.c_void_p(0x1000), ctypes.c_void_p(0x2000)
    assert L.cn_smem_book(k1, 0, 100 * 1024, 0) == 1  # asked without committing: still to do
    assert L.cn_smem_book(k1, 0, 100 * 1024, 1) == 1
    assert L.cn_smem_book(k1, 0, 100 * 1024, 1) == 0  # covered now
    assert L.cn_smem_book(k1, 0, 64 * 1024, 1) == 0   # a smaller size is covered by the larger
    assert L.cn_smem_book(k1, 0, 200 * 1024, 1) == 1  # a larger one is not
    assert L.cn_smem_book(k1, 1, 100 * 1024, 1) == 1  # another device: its own call
    assert L.cn_smem_book(k2, 0, 100 * 1024, 1) == 1  # another kernel: its own call
    assert L.cn_smem_book(k1, 1, 100 * 1024, 1) == 0
