"""The C-ABI library loads and exports exactly what include/lsa_b200.h declares (no compute, so no GPU needed)."""

import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared_functions():
    text = open(os.path.join(ROOT, "include", "lsa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lsa_[a-z0-9_]+)\s*\(", text)))


def test_the_library_exports_every_declared_entry_point():
    from lsa_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/lsa_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "the ctypes binding and the header name different entry points"


def test_error_codes_have_names_and_size_queries_answer_without_a_gpu():
    from lsa_b200 import _lib

    lib = _lib.load()
    assert lib.lsa_abi_version() == _lib.ABI_VERSION
    for code in range(-6, 1):
        assert lib.lsa_error_string(code)
    assert b"unknown" in lib.lsa_error_string(-99)
    assert _lib.query("lsa_sparse_attend_workspace_bytes", 4, 40, 128, 1) == 0
    assert _lib.query("lsa_sparse_attend_workspace_bytes", 4, 40, 128, 8) == 8 * 4 * 40 * 129 * 4
    assert _lib.query("lsa_flat_select_decode_workspace_bytes", 64, 32, 4) == 64 * 32 * 4 * 8


def test_arguments_are_refused_on_the_host_before_any_launch():
    from lsa_b200 import _lib

    lib = _lib.load()
    # NULL pointers and bad sizes are decided before the CUDA runtime is touched
    assert lib.lsa_pool_keys(None, 0, 4, 4, 16, None, None) == -2
    assert lib.lsa_ward_merge(None, None, 4.0, 1, 64, 64, 32, 64.0, 256, None, None, None, None, 0, None) == -2
    assert lib.lsa_lse_merge(None, 0, None, 2, 8, 128, None, None, None, None) == -2
    with pytest.raises(ValueError, match="NULL"):
        _lib.call("lsa_expand", None, 1, 1, None, None, 0, 1, None, None, 1, 0, 1, None, 0, 0, 1, 1, 1, 0, 0, None, None,
                  None, None)
