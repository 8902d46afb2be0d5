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


def test_op_wrappers_reject_inconsistent_shapes_before_any_launch():
    """The kernels take shapes on trust; the Python wrappers check them first (no GPU needed to see the errors)."""
    from types import SimpleNamespace
    import pytest
    import torch
    from neuralattentionsearchlinear_b200 import _ops
    tb = SimpleNamespace(types_i=torch.zeros(2, 4, 2, 2, dtype=torch.int32), T=256, nats_block_size=64)
    q = torch.zeros(2, 256, 4, 64)
    with pytest.raises(ValueError, match="CUDA device"):
        _ops._check_qkv(q, q, q, tb, "test", same_heads=True)
    fake = lambda *s: SimpleNamespace(shape=torch.Size(s), dim=lambda: len(s), is_cuda=True, device="cuda:0")
    tbc = SimpleNamespace(types_i=SimpleNamespace(shape=torch.Size((2, 4, 2, 2)), device="cuda:0"))
    _ops._check_qkv(fake(2, 256, 4, 64), fake(2, 256, 4, 64), fake(2, 256, 4, 32), tbc, "ok", same_heads=True)
    _ops._check_qkv(fake(2, 128, 4, 64), fake(2, 256, 2, 64), fake(2, 256, 2, 32), tbc, "ok", same_heads=False)
    for bad in [(fake(2, 256, 4, 64), fake(3, 256, 4, 64), fake(2, 256, 4, 64)),          # batch
                (fake(2, 256, 4, 64), fake(2, 256, 4, 32), fake(2, 256, 4, 64)),          # head dim of q vs k
                (fake(2, 256, 4, 64), fake(2, 256, 4, 64), fake(2, 128, 4, 64)),          # k vs v length
                (fake(2, 256, 4, 64), fake(2, 200, 4, 64), fake(2, 200, 4, 64))]:         # q vs k length (linear)
        with pytest.raises(ValueError):
            _ops._check_qkv(*bad, tbc, "bad", same_heads=True)
    with pytest.raises(ValueError, match="query heads"):
        _ops._check_qkv(fake(2, 256, 5, 64), fake(2, 256, 2, 64), fake(2, 256, 2, 64), tbc, "bad", same_heads=False)
