"""The C ABI: the library loads without a GPU and exports exactly what include/daceml_b200.h declares."""
import ctypes
import os
import re

import pytest
import torch

from daceml_b200 import build as builder
from daceml_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def library():
    builder.build()
    return L.load_library()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "daceml_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200ml_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(library):
    declared = declared_symbols()
    assert declared, "no declarations found in the header"
    assert sorted(L.EXPORTED_SYMBOLS) == declared


def test_every_declared_symbol_is_exported(library):
    for name in declared_symbols():
        assert hasattr(library, name), f"{name} is declared in the header but not exported"


def test_struct_layouts_match_header():
    # field order of the ctypes mirrors follows the header; sizes are what a C compiler produces
    assert ctypes.sizeof(L.GemmParams) == 4 * 4 + 17 * 8 + 4 * 4 + 5 * 8 + 2 * 8 + 2 * 4
    assert ctypes.sizeof(L.ConvParams) == 2 * 4 + 16 * 8 + 7 * 8
    assert ctypes.sizeof(L.AttentionParams) == 17 * 8 + 2 * 4 + 5 * 8


def test_version_and_error_string(library):
    assert library.b200ml_version() >= 100
    assert isinstance(library.b200ml_last_error(), bytes)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_gpu_fails_loudly(library):
    with pytest.raises(L.B200Error) as e:
        L.Context(0)
    assert "no CPU path" in str(e.value)
    import daceml_b200.onnx as donnx
    x = torch.zeros(4, 4)
    with pytest.raises(RuntimeError):
        donnx.ONNXRelu(X=x, Y=torch.zeros(4, 4))


def test_null_context_is_rejected(library):
    rc = library.b200ml_softmax(None, 0, None, None, None, 1, 1, 1, ctypes.c_float(1.0), 0, None)
    assert rc == L.ERR_INVALID
    assert b"null context" in library.b200ml_last_error()
