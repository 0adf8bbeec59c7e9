"""The C-ABI library loads on a machine without a GPU and exports what include/rsfa.h declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "rsfa.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"RSFA_API\s+[\w\s\*]+?\b(rsfa_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("rsfa_fwd", "rsfa_fwd_host", "rsfa_get_tiling", "rsfa_select_path", "rsfa_sm_count",
                 "rsfa_device_status", "rsfa_strerror", "rsfa_version"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from ascend_rsfa import _capi

    lib = ctypes.CDLL(_capi.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name
        assert name in _capi.SIGNATURES, "binding missing for " + name
    assert set(_capi.SIGNATURES) == set(declared_functions())


def test_no_compute_calls_needed_for_metadata():
    from ascend_rsfa import _capi

    lib = _capi.load()
    assert lib.rsfa_version() >= 100
    assert _capi.strerror(0) == "ok"
    assert "invalid" in _capi.strerror(_capi.RSFA_ERR_INVALID_ARGUMENT)
    assert lib.rsfa_launch_count() == 0 or lib.rsfa_launch_count() > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ascend_rsfa import _capi

    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _capi.load()
