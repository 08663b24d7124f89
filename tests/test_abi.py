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


def test_null_arguments_are_refused_before_any_device_work():
    """Entry points validate their pointers first: a null handle or buffer gives AB2_ERR_BAD_ARG
    (-7) and a message, on a machine without a GPU as well."""
    p = pkg()
    calls = {
        "ab2_qlinear_forward": (None, None, 1, 2, None, None),
        "ab2_qweight_dequant": (None, None, 0, None),
        "ab2_swiglu": (None, None, None, 8, 2, None),
        "ab2_model_decode_step": (None, None, None, 0, 1, None, None, None),
        "ab2_model_decode_step_host": (None, None, None, 0, 1, None, None),
        "ab2_device_status": (None,),
    }
    for name, args in calls.items():
        assert getattr(p.lib, name)(*args) == -7, name
        assert b"null" in p.lib.ab2_last_error(), name
