"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with an error code before touching a device."""

import ctypes
import os
import re

import pytest

from flashomni_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            names += re.findall(r"FO_API\s+[\w\s\*]+?\b(fo_\w+)\s*\(", text)
    return names


def test_library_loads_and_exports_every_declared_symbol():
    lib = _native.load()
    declared = _declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert set(declared) == set(_native.SIGNATURES), "ctypes prototypes and header differ"
    assert lib.fo_abi_version() == 2


def test_argument_errors_are_reported_not_raised_as_faults():
    lib = _native.load()
    assert lib.fo_packbits(None, 8, 1, None, None) == _native.FO_ERR_INVALID_ARG
    assert b"null" in lib.fo_last_error()
    assert lib.fo_packbits(None, 0, 1, None, None) == _native.FO_OK
    assert lib.fo_gemm_q(None, None, None, None, 1, 1, 128, 128, 64, 1, 0, 128, 128, 0, 1, None, 0, None, None,
                         0, None) == _native.FO_ERR_INVALID_ARG
    rc = lib.fo_sparse_attn_fwd(*([None] * 5), 1, 128, 128, 1, 1, 128, 128, 128, 128, 128, 128, 128, 128, 128,
                                128, 128, *([None] * 3), 1, None, None, 0, 0, ctypes.c_float(1.0), None, None)
    assert rc == _native.FO_ERR_INVALID_ARG
    assert lib.fo_gemm_workspace_bytes(1, 128, 128, 128, 128) >= 64
    assert lib.fo_mask_compact_scratch_bytes(10, 3) >= 10 * 16


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("FLASHOMNI_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(RuntimeError, match="native library not found"):
        _native.load()
