"""The C-ABI library loads on a CPU-only machine, exports every symbol the
header declares, and refuses to compute without a GPU (no CPU fallback)."""
import ctypes as C
import os
import re

import pytest

from nnv_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nnvb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nnvb_[A-Za-z_0-9]+)\s*\(", text)))


def test_header_symbols_exported_and_bound():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), "symbol %s declared in nnvb200.h is not exported" % n
        assert n in _lib.SIGNATURES, "symbol %s has no ctypes signature" % n
    for n in _lib.SIGNATURES:
        assert n in names, "ctypes binds %s which the header does not declare" % n


def test_abi_version_and_strerror():
    lib = _lib.load()
    assert lib.nnvb_abi_version() == 2
    assert lib.nnvb_strerror(0) == b"ok"
    assert b"arena" in lib.nnvb_strerror(_lib.NNVB_E_CAPACITY)


def test_layer_desc_layout():
    # offsets the C compiler gives nnvb_layer_desc on x86-64
    assert _lib.LayerDesc.W.offset == 64
    assert _lib.LayerDesc.bn_eps.offset == 112
    assert _lib.LayerDesc.avgpool_divisor.offset == 120
    assert C.sizeof(_lib.LayerDesc) == 128
    assert C.sizeof(_lib.Opts) == 32
    assert C.sizeof(_lib.ReluStats) == 32


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    h = C.c_void_p()
    s = lib.nnvb_init(0, 0, C.byref(h))
    assert s == _lib.NNVB_E_CUDA and not h.value
    assert b"no CPU path" in lib.nnvb_last_error()
    from nnv_b200.engine import Context
    with pytest.raises(_lib.NNVError):
        Context(0)


def test_null_arguments_are_rejected():
    lib = _lib.load()
    assert lib.nnvb_net_create(None, None, 0, 1, 1, 1, None) == _lib.NNVB_E_ARG
    assert lib.nnvb_batch_create(None, 1, None) == _lib.NNVB_E_ARG
    assert lib.nnvb_destroy(None) == _lib.NNVB_OK
    assert lib.nnvb_net_destroy(None) == _lib.NNVB_OK
    assert lib.nnvb_batch_destroy(None) == _lib.NNVB_OK


def test_mex_gateway_compiles_against_stub_header():
    # the MEX gateway is shipped as source; check that it is valid C++ against the documented MEX API
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    src = os.path.join(ROOT, "nnv_b200", "csrc", "nnvb200_mex.cpp")
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-I", os.path.join(ROOT, "include", "mex_stub"), src],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
