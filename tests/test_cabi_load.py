"""The C-ABI library loads and exports every symbol include/b2c.h declares; host-side argument
checking returns status codes without touching a device (CPU only)."""
import ctypes
import os
import re

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from pydtnn_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return _lib


def test_every_declared_symbol_is_exported_and_bound(lib):
    header = open(os.path.join(REPO, "include", "b2c.h")).read()
    declared = set(re.findall(r"\b(b2c_[a-z0-9_]+)\s*\(", header))
    declared -= {"b2c_status", "b2c_conv_desc", "b2c_bn_params"}
    assert len(declared) >= 24
    handle = ctypes.CDLL(lib.LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/b2c.h but not exported"
    assert declared == set(lib.PROTOTYPES), declared ^ set(lib.PROTOTYPES)


def test_status_strings(lib):
    L = lib.lib()
    assert L.b2c_status_string(0) == b"ok"
    for s in range(-9, 0):
        assert len(L.b2c_status_string(s)) > 3
    assert L.b2c_version() >= 100


def _desc(lib, **kw):
    base = dict(layout=0, dtype=0, w_layout=0, engine=0, n=2, h=8, w=8, ci=3, co=4, kh=3, kw=3, vpad=1, hpad=1,
                vstr=1, hstr=1, vdil=1, hdil=1)
    base.update(kw)
    return lib.ConvDesc(**base)


def test_argument_validation_is_host_side(lib):
    L = lib.lib()
    d = _desc(lib)
    assert L.b2c_conv_fprop(ctypes.byref(d), None, None, None, None, 0, None, None, 0, None) == -1
    assert L.b2c_conv_fprop(None, None, None, None, None, 0, None, None, 0, None) == -1
    assert L.b2c_conv_dgrad(ctypes.byref(_desc(lib, vstr=0)), None, None, None, None, 0, None) == -2
    assert L.b2c_conv_wgrad(ctypes.byref(_desc(lib, layout=7)), None, None, None, None, None, 0, None) == -3
    # filter larger than the padded input: empty output
    assert L.b2c_conv_fprop(ctypes.byref(_desc(lib, h=2, w=2, kh=5, kw=5, vpad=0, hpad=0)),
                            None, None, None, None, 0, None, None, 0, None) == -2
    assert L.b2c_conv_engine_for(ctypes.byref(d), 0) in (lib.ENGINE_FMA, lib.ENGINE_TENSOR)
    assert L.b2c_conv_engine_for(ctypes.byref(d), 5) == -3
    assert L.b2c_relu_forward(0, 16, None, None, None) == -1
    assert L.b2c_sgd_update(3, 16, None, None, None, 0.1, 0.9, 0.0, 0, None) == -3
    with pytest.raises(lib.B2CError):
        lib.check(-2)


def test_workspace_query(lib):
    L = lib.lib()
    # wgrad reduces over n*ho*wo with few output tiles: split-K partials + bias-gradient partials
    d = _desc(lib, n=64, h=32, w=32, ci=64, co=64, engine=lib.ENGINE_FMA)
    assert L.b2c_conv_workspace_bytes(ctypes.byref(d), lib.PASS_WGRAD) > 0
    assert L.b2c_conv_workspace_bytes(ctypes.byref(_desc(lib, n=0)), lib.PASS_FPROP) == 0
