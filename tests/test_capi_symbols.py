"""CPU tests of the drop-in boundary: the built C-ABI library loads and exports every entry point the header declares."""
import ctypes
import os
import re

import pytest

from deepscalemd_b200 import build, capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def library():
    build.build()          # nvcc cross-compiles for sm_100a without a GPU
    return ctypes.CDLL(capi.LIBRARY)


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dsmd_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsmd_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(capi.SYMBOLS)


def test_every_declared_symbol_is_exported(library):
    for name in declared_symbols():
        assert hasattr(library, name), name


def test_missing_library_is_an_error_not_a_fallback(monkeypatch):
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIBRARY", os.path.join(ROOT, "deepscalemd_b200", "no_such_library.so"))
    with pytest.raises(ImportError):
        capi.load()


def test_product_does_not_reach_the_oracle():
    """Nothing in the package, the headers or the build imports or links the oracle."""
    for folder in ("deepscalemd_b200", "include"):
        for base, _, files in os.walk(os.path.join(ROOT, folder)):
            for f in files:
                if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h", ".cpp")):
                    text = open(os.path.join(base, f)).read()
                    assert "cpu_oracle" not in text and "dsmd_oracle" not in text and "oracle/" not in text, f


def test_adapter_check_library_resolves_every_symbol():
    """The C++ adapters compiled against the reference's headers (oracle/_ref/libdsmd_adapter_check.so, what the GPU
    adapter tests drive) load without an unresolved symbol: no compute call is made."""
    import ctypes
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(here, "oracle", "_ref", "libdsmd_adapter_check.so")
    if not os.path.exists(path):
        import pytest
        pytest.skip("adapter check library not built (needs the reference headers)")
    ctypes.CDLL(path, mode=os.RTLD_NOW)
