"""The C-ABI library builds, loads and exports every symbol the public header declares
(no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

from neuralattentionsearchlinear_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            src = open(os.path.join(inc, f)).read()
            src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
            names += re.findall(r"\b(natsl_\w+)\s*\(", src)
    return sorted(set(names))


def test_library_builds_and_exports_all_declared_symbols():
    path = build.build_library()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    declared = _declared()
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert set(_lib.PROTOTYPES) | {"natsl_last_error"} == set(declared)


def test_abi_version_and_error_string():
    lib = _lib.load()
    assert lib.natsl_abi_version() == 1
    # argument validation happens on the host before any CUDA call
    st = lib.natsl_build_tables(None, 1, 1, 1, 1, 64, 64, 128, None, None, None, None, None, None, None, None, None)
    assert st == -3 and b"null" in lib.natsl_last_error()
    st = lib.natsl_chunk_local_cumsum(None, None, 1, 1, 1, None)
    assert st == -3
