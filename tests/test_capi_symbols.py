"""The C-ABI library must build, load without a GPU, and export every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sharpnet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(snb200_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(built_library):
    lib = ctypes.CDLL(built_library)
    names = _declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/sharpnet_b200.h but not exported"


def test_binding_table_matches_header(built_library):
    from sharpnet_b200 import _capi
    assert sorted(_capi.SIGNATURES) == _declared_symbols()
    lib = _capi.load()
    assert lib.snb200_get_version() >= 100


def test_reference_side_binding_names_every_entry_point():
    # the P/Invoke class a SharpNet maintainer would add declares every symbol of the header
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    missing = [n for n in _declared_symbols() if ("extern cublasStatus_t " + n + "(") not in text
               and ("extern int " + n + "(") not in text and ("extern long " + n + "(") not in text
               and ("extern IntPtr " + n + "(") not in text]
    assert not missing, missing


def test_create_fails_loudly_without_a_device(built_library):
    import torch
    if torch.cuda.is_available():
        return
    from sharpnet_b200 import _capi
    lib = _capi.load()
    h = ctypes.c_void_p()
    assert lib.snb200_create(ctypes.byref(h), 0) != 0       # no CPU fallback
    assert not h.value
    assert lib.snb200_gemm(None, 0, 0, 1, 1, 1, 1, 1.0, None, None, 0.0, None) == 1   # NOT_INITIALIZED
    import pytest
    from sharpnet_b200.tensor import GPUWrapper
    with pytest.raises(RuntimeError):
        GPUWrapper(0)


def test_activation_codes_agree_everywhere():
    """The activation selector has one numbering -- cudnnActivationMode_t of the reference
    (Prod/GPU/CudnnWrapper.cs:267-281) -- in the C header, the ctypes binding, the oracle and the C++ mirror."""
    import re
    from oracle import sharpnet_oracle as orc
    from sharpnet_b200 import _capi
    header = open(os.path.join(ROOT, "include", "sharpnet_b200.h")).read()
    mirror = open(os.path.join(ROOT, "sharpnet_b200", "host", "sharpnet_tensor.hpp")).read()
    expected = {"SIGMOID": 0, "RELU": 1, "TANH": 2, "CLIPPED_RELU": 3, "ELU": 4, "IDENTITY": 5, "SWISH": 6, "SOFTMAX": 1000,
                "LEAKY_RELU": 1002, "LN": 1004}
    for name, value in expected.items():
        m = re.search(r"SNB200_ACT_%s\s*=\s*(\d+)" % name, header)
        assert m and int(m.group(1)) == value, name
        assert getattr(_capi, "ACT_" + name) == value, name
        assert getattr(orc, "ACT_" + name) == value, name
        m = re.search(r"CUDNN_ACTIVATION_%s\s*=\s*(\d+)" % name, mirror)
        assert m and int(m.group(1)) == value, name
