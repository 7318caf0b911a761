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
    assert ctypes.sizeof(L.ConvParams) == 2 * 4 + 16 * 8 + 8 * 8
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


@pytest.mark.gpu
def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_context_usable():
    """The give-up path of the library's device-side waits, run on purpose: a CTA waits 2 ms on an mbarrier nothing
    completes, records its code and returns.  The status call reports it once, clears the word, and a GEMM launched
    afterwards on the same context is correct.  No trap, no fault, nothing left waiting."""
    import numpy as np
    from daceml_b200 import kernels as K
    ctx = L.get_context(0)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0
    waited = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(ctx.lib.b200ml_wait_probe(ctx.handle, 2_000_000, ctypes.c_void_p(waited.data_ptr()), L.current_stream()))
    torch.cuda.synchronize()
    with pytest.raises(L.B200Error) as err:
        ctx.device_status()
    assert err.value.code == L.ERR_DEVICE and "status 6" in str(err.value)
    assert 2000 <= int(waited) < 50_000, int(waited)  # it waited the 2 ms it was given, not the default second
    assert ctx.device_status() == 0, "the status word was not cleared"
    # limits outside 1 ns .. 100 ms are refused on the host
    assert ctx.lib.b200ml_wait_probe(ctx.handle, 10**10, None, L.current_stream()) == L.ERR_INVALID
    rng = np.random.default_rng(0)
    a = torch.from_numpy(rng.standard_normal((256, 512)).astype(np.float32)).half().cuda()
    b = torch.from_numpy(rng.standard_normal((512, 384)).astype(np.float32)).half().cuda()
    y = torch.empty(256, 384, dtype=torch.float16, device="cuda")
    K.gemm(a, b, y)
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)
    assert ctx.device_status() == 0
