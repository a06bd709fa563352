"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import os
import re

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "lmoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lmoe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from swamla_b200 import _cabi, build
    build.build()
    lib = _cabi.load()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/lmoe.h but not exported"
        assert name in _cabi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_cabi.SIGNATURES) == set(declared)


def test_version_and_status_strings():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    assert lib.lmoe_version() == 1
    assert _cabi.status_string(0) == "ok"
    assert "shape" in _cabi.status_string(-2)
    assert "timed out" in _cabi.status_string(102)


def test_host_side_shape_helpers():
    from swamla_b200 import _cabi
    lib = _cabi.load()
    s = _cabi.Shape(T=1024, D=1024, L=256, E=128, K=12, F=256, Fs=1024, n_shared=1)
    assert lib.lmoe_padded_rows(s) == 1024 * 12 + 128 * 128
    assert lib.lmoe_route_workspace_bytes(s) == ((1024 * 12 + 255) // 256) * 128 * 4
    bad = _cabi.Shape(T=1024, D=1024, L=256, E=512, K=12, F=256, Fs=1024, n_shared=1)
    assert lib.lmoe_padded_rows(bad) == 0
