"""CPU tests of the C-ABI library: it loads, exports every declared symbol, and refuses to compute
without a device.  No compute call is made here."""
import ctypes
import os
import re

import pytest

import attention_superoptimizer_b200 as mg
from attention_superoptimizer_b200 import _abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mgd?_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_abi.LIB_PATH)
    for header in ("mugraph.h", "mugraph_device.h"):
        names = declared_symbols(header)
        assert len(names) > 20
        for name in names:
            assert hasattr(lib, name), "%s declares %s but the library does not export it" % (header, name)


def test_python_binding_covers_the_header():
    assert sorted(_abi.SIGNATURES) == declared_symbols("mugraph.h")


def test_struct_layouts_match_the_headers():
    # sizes the C side static-checks by construction: 4+4+4+16+4+4 (+pad) +8+8
    assert ctypes.sizeof(_abi.mg_tensor) == 56
    assert ctypes.sizeof(_abi.mgd_op) == 80
    assert ctypes.sizeof(_abi.mgd_program) == 48 + 24 * 80


def test_no_device_is_reported_not_hidden():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _abi.load()
    h = ctypes.c_void_p()
    st = lib.mg_runtime_create(0, 1 << 20, ctypes.byref(h))
    assert st == 7 and h.value is None  # MG_ERR_NO_DEVICE: there is no CPU fallback
    assert lib.mg_last_error()


def test_null_and_bad_arguments_return_status_codes():
    lib = _abi.load()
    assert lib.mg_runtime_create(0, 0, None) == 1
    assert lib.mg_graph_create(None, None) == 1
    assert lib.mg_graph_destroy(None) == 1
    assert lib.mg_op_fingerprint(None, 0) == 1
    assert lib.mg_version().startswith(b"mugraph")
