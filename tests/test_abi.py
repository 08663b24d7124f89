"""The C-ABI library loads and exports every symbol the header declares (no GPU)."""
import ctypes
import os
import re

from helpers import ROOT, pkg


def declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(ab2_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    p = pkg()
    lib = ctypes.CDLL(p._lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 15
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"missing exports: {missing}"


def test_binding_declares_every_symbol():
    p = pkg()
    assert sorted(p._lib.SIGNATURES) == declared_symbols()


def test_version_and_error_string():
    p = pkg()
    assert p.lib.ab2_version() >= 100
    assert isinstance(p.lib.ab2_last_error(), bytes)
