"""The C-ABI library loads and exports every symbol include/grab_anns.h declares (no GPU)."""
import ctypes
import importlib
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    out = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        out += re.findall(r"\b(grab_[a-z0-9_]+)\s*\(", text)
    return sorted(set(out))


def test_header_symbols_exported():
    grab = importlib.import_module("grab-anns_b200")
    grab.build()
    lib = ctypes.CDLL(grab.LIB_PATH)
    syms = _declared_symbols()
    assert len(syms) >= 20
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing


def test_status_strings_and_version():
    grab = importlib.import_module("grab-anns_b200")
    lib = grab.lib()
    assert lib.grab_abi_version() == 3
    assert lib.grab_status_string(0) == b"ok"
    assert lib.grab_status_string(1) == b"invalid argument"


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    grab = importlib.import_module("grab-anns_b200")
    monkeypatch.setattr(grab, "_lib", None)
    monkeypatch.setattr(grab, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        grab.lib()
    except grab.GrabError as e:
        assert "missing" in str(e)
    else:
        raise AssertionError("loading a missing extension must raise")
