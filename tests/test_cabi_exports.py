"""CPU-side checks of the drop-in boundary: the shared library loads and exports every entry
point that include/dyb200.h declares, and there is no silent fallback without a GPU."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from dynet_b200 import build
    return build.build()


def declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "dyb200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(dyb200_[a-z0-9_]+)\s*\(", hdr)))


def test_every_declared_symbol_is_exported(built):
    import ctypes
    L = ctypes.CDLL(built)
    syms = declared_symbols()
    assert len(syms) >= 45
    missing = [s for s in syms if not hasattr(L, s)]
    assert not missing, missing


def test_binding_table_matches_header(built):
    from dynet_b200 import capi
    assert sorted(capi.exported_symbols()) == declared_symbols()


def test_no_cpu_fallback_without_gpu(built):
    import torch
    from dynet_b200 import capi
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(capi.Dyb200Error):
        capi.Context(0)


def test_every_binding_declares_its_argument_types(built):
    """ctypes passes a Python int as a 32-bit C int unless argtypes says otherwise: a device pointer given to an
    undeclared function is truncated.  Every entry point the binding exposes must therefore carry argtypes."""
    from dynet_b200 import capi
    L = capi.lib()
    no_args = {"dyb200_version"}
    untyped = [s for s in capi.exported_symbols() if s not in no_args and getattr(L, s).argtypes is None]
    assert not untyped, untyped
