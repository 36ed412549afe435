"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol that
include/vexact_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "vexact_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared_symbols()
    assert "b200_gemm_bf16" in names and "b200_paged_attn_fwd" in names and len(names) >= 15


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/vexact_b200.h but not exported"


def test_ctypes_signatures_cover_header(lib):
    from vexact_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    assert lib.b200_abi_version() == _lib.ABI_VERSION == 4


def test_argument_validation_without_gpu(lib):
    # NULL pointers are rejected on the host before anything touches a device.
    assert lib.b200_rmsnorm(None, None, None, 1, 8, 8, 8, ctypes.c_float(1e-6), 0, None) == -1
    assert lib.b200_gemm_bf16(None, None, None, None, 1, 8, 8, 8, 8, 8, 0, None) == -1
    assert lib.b200_kv_store(None, None, None, None, None, 1, 1, 8, 8, 8, 8, 1, None) == -1


def test_no_product_import_of_oracle():
    """The package must not reach into oracle/ (the oracle is test infrastructure)."""
    pkg = os.path.join(ROOT, "vexact_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(".py"):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f


def test_library_carries_the_hash_of_its_sources(lib):
    """The loader binds argument lists by position, so a library built from other sources must be
    refused: the hash compiled into the binary has to equal the hash of the sources beside it."""
    import ctypes as C

    from vexact_b200 import _lib, build

    text = open(os.path.join(ROOT, "include", "vexact_b200.h")).read()
    assert re.search(r"const\s+char\s*\*\s*b200_source_hash\s*\(", text)
    fn = lib.b200_source_hash
    fn.restype = C.c_char_p
    assert fn().decode() == build._source_hash() == build.built_hash()

    class Stale:
        class b200_source_hash:  # noqa: N801  (stands in for the ctypes function object)
            restype = None

            def __new__(cls):
                return b"0" * 64

    import pytest

    with pytest.raises(_lib.B200Error, match="other sources"):
        _lib._check_fresh(Stale)
