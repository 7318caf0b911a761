"""The allocation-free reduction entry point, b200ml_reduce_static.

It serves callers that must not allocate device memory (code under CUDA-graph capture or inside a
serving loop, plug-ins with a fixed memory budget): its scratch is an array built into the library.
The test calls it through the C ABI, without creating a context for it, and checks it against the
ordinary entry point (b200ml_reduce, context scratch) twice in a row with different data, so a stale
partial left in the shared array by the first call would show up in the second.

The file name sorts last on purpose: pytest runs it after every other test file.
"""
import ctypes

import pytest
import torch

from daceml_b200 import lib as L

pytestmark = pytest.mark.gpu


def _static(x, y, op, outer, red, inner):
    lib = L.load_library()
    rc = lib.b200ml_reduce_static(L.dtype_code(x.dtype), op, L.ptr(x), L.ptr(y), outer, red, inner, L.current_stream(x.device))
    L.check(rc)


def _with_context(x, y, op, outer, red, inner):
    ctx = L.get_context(x.device)
    L.check(ctx.lib.b200ml_reduce(ctx.handle, L.dtype_code(x.dtype), op, L.ptr(x), L.ptr(y), outer, red, inner,
                                  L.current_stream(x.device)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_static_reduce_matches_context_reduce_twice_in_a_row(dtype):
    torch.cuda.set_device(0)
    gen = torch.Generator("cuda").manual_seed(11)
    # rows long enough to be cut into slices, so both calls really go through the scratch array
    cases = [(L.RED_SUM, 3, 1_200_000), (L.RED_MAX, 2, 900_000)]
    for op, outer, red in cases:
        x = (torch.randn(outer, red, device="cuda", generator=gen) * 0.25).to(dtype)
        got = torch.full((outer, ), -7.0, dtype=dtype, device="cuda")
        ref = torch.full((outer, ), 7.0, dtype=dtype, device="cuda")
        _static(x, got, op, outer, red, 1)
        _with_context(x, ref, op, outer, red, 1)
        torch.cuda.synchronize()
        tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)
        torch.testing.assert_close(got.float(), ref.float(), **tol)
        exact = x.float().sum(1) if op == L.RED_SUM else x.float().amax(1)
        torch.testing.assert_close(got.float(), exact, rtol=2e-2 if dtype == torch.float16 else 1e-3, atol=0.5)


def test_static_reduce_short_rows_and_columns():
    torch.cuda.set_device(0)
    x = torch.randn(6, 50, 7, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    got, ref = torch.empty(6, 7, device="cuda"), torch.empty(6, 7, device="cuda")
    _static(x, got, L.RED_MEAN, 6, 50, 7)
    _with_context(x, ref, L.RED_MEAN, 6, 50, 7)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)


def test_static_reduce_rejects_what_does_not_fit():
    torch.cuda.set_device(0)
    # 550 long rows are cut into two slices each: 1100 partial results, more than the 1024 of the built-in array
    outer, red = 550, 8192
    x = torch.ones(outer, red, dtype=torch.float32, device="cuda")
    y = torch.empty(outer, dtype=torch.float32, device="cuda")
    lib = L.load_library()
    rc = lib.b200ml_reduce_static(L.F32, L.RED_SUM, L.ptr(x), L.ptr(y), outer, red, 1, L.current_stream(x.device))
    assert rc == L.ERR_WORKSPACE
    assert b"built-in scratch" in lib.b200ml_last_error()
    # the ordinary entry point serves the same request from its context's buffer
    _with_context(x, y, L.RED_SUM, outer, red, 1)
    torch.cuda.synchronize()
    assert float(y.min()) == float(y.max()) == float(red)
