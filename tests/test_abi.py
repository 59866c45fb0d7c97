"""The C-ABI library: it loads without a GPU and exports every symbol the header declares."""
import ctypes
import importlib
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(nsa_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    build = importlib.import_module("openbox-llm_b200.build")
    path = build.build_library()
    handle = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(handle, name), name


def test_binding_table_matches_header():
    L = importlib.import_module("openbox-llm_b200._lib")
    assert set(L.SIGNATURES) == _declared()
    lib = L.lib()
    assert lib.nsa_version() >= 100
    # argument checking happens on the host, before any CUDA call
    d = L.dims(1, 3, 2, 16, 64, L.DTYPE_BF16)
    assert lib.nsa_range_attn_fwd(None, None, None, None, None, d, 16, 0, 8, 0, 0, None) == -1
    assert b"multiple" in lib.nsa_last_error()
    d = L.dims(1, 4, 2, 16, 48, L.DTYPE_BF16)
    assert lib.nsa_selection_fwd(None, None, None, None, None, None, d, 4, 16, None, 0, 0, None) == -1
    d = L.dims(1, 4, 2, 16, 64, L.DTYPE_BF16)
    assert lib.nsa_selection_fwd(None, None, None, None, None, None, d, 4, 8, None, 0, 0, None) == -1
    assert lib.nsa_tc_supported(L.dims(1, 4, 2, 16, 64, L.DTYPE_F32), 64) == 0
    assert lib.nsa_csr_workspace_bytes(2, 2, 128, 4, 16) > 0


def test_missing_library_fails_loudly(monkeypatch):
    L = importlib.import_module("openbox-llm_b200._lib")
    monkeypatch.setattr(L, "_lib", None)
    monkeypatch.setattr(L, "LIB_PATH", "/nonexistent/libnsa_b200.so")
    try:
        L.lib()
    except L.NsaError as e:
        assert "no non-CUDA fallback" in str(e)
    else:
        raise AssertionError("expected NsaError")


def test_product_does_not_import_oracle():
    pk = os.path.join(ROOT, "openbox-llm_b200")
    for dirpath, _, files in os.walk(pk):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, os.path.join(dirpath, f)
