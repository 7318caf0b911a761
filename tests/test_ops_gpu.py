"""Per-operator parity on the B200: the CUDA path (through the donnx frontend and the C ABI) against
the CPU oracle and the committed golden vectors.  Shapes follow the reference's own tests
(tests/pure_expansions/test_expansions.py, test_conv_expansion.py) plus ragged and empty cases."""
import os

import numpy as np
import pytest
import torch

import daceml_b200.onnx as donnx
from daceml_b200 import kernels as K, lib as L, sdfg as sd
from oracle import ops
from conftest import assert_close

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DTYPES = [torch.float32, torch.float16]


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).cuda()


def rounded(a, dtype):
    """The oracle sees inputs already rounded to the storage type."""
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).float().numpy()


def empty(shape, dtype):
    return torch.empty(shape, dtype=dtype, device="cuda")


def status_ok():
    torch.cuda.synchronize()
    assert L.get_context(0).device_status() == 0


# ------------------------------------------------------------------------------------------------
# MatMul / Gemm / Einsum
# ------------------------------------------------------------------------------------------------
def test_matmul_expansion_reference_test():
    """tests/pure_expansions/test_expansions.py:23-63, written against the same SDFG API."""
    g = gold("matmul")
    X, Z = g["a"], g["b"]
    sdfg = sd.SDFG("matmul_expansion")
    sdfg.add_array("X", X.shape, np.float32)
    sdfg.add_array("Z", Z.shape, np.float32)
    sdfg.add_array("__return", g["y"].shape, np.float32)
    state = sdfg.add_state()
    access_X, access_Z, access_result = state.add_access("X"), state.add_access("Z"), state.add_access("__return")
    op_node = donnx.ONNXMatMul("Matmul")
    state.add_node(op_node)
    state.add_edge(access_X, None, op_node, "A", sdfg.make_array_memlet("X"))
    state.add_edge(access_Z, None, op_node, "B", sdfg.make_array_memlet("Z"))
    state.add_edge(op_node, "Y", access_result, None, sdfg.make_array_memlet("__return"))
    sdfg.expand_library_nodes()
    assert any(isinstance(n, sd.KernelTasklet) for n, _ in sdfg.all_nodes_recursive())
    result = sdfg(X=X, Z=Z)
    assert_close(result, g["y"], torch.float32, what="matmul golden")
    status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("a_shape, b_shape", [((2, 4), (4, 3)), ((3, 5, 8), (8, 6)), ((2, 3, 16, 8), (2, 3, 8, 24)),
                                              ((130, 72), (72, 136)), ((8, 64, 256), (256, 512)), ((2, 4, 128, 64), (2, 4, 64, 128)),
                                              ((5, 40), (3, 40, 24)), ((1, 8), (8, 1))])
def test_matmul_shapes(dtype, a_shape, b_shape, rng):
    a, b = rng.standard_normal(a_shape).astype(np.float32), rng.standard_normal(b_shape).astype(np.float32) * 0.2
    ref = ops.matmul(rounded(a, dtype), rounded(b, dtype))
    y = empty(ref.shape, dtype)
    donnx.ONNXMatMul(A=dev(a, dtype), B=dev(b, dtype), Y=y)
    assert_close(y, ref, dtype, what=f"matmul {a_shape}x{b_shape}")
    status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k", [(256, 512, 1024), (4096, 256, 64), (1000, 520, 264), (128, 64, 512), (300, 3072, 128)])
def test_matmul_tensor_core_shapes(dtype, m, n, k, rng):
    """Sizes that take the tcgen05 path in fp16 (all three tile widths, ragged edges, K not a multiple of 64)."""
    a, b = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32) * 0.05
    ref = ops.matmul(rounded(a, dtype), rounded(b, dtype))
    y = empty((m, n), dtype)
    donnx.ONNXMatMul(A=dev(a, dtype), B=dev(b, dtype), Y=y)
    assert_close(y, ref, dtype, what=f"matmul {m}x{n}x{k}")
    status_ok()


@pytest.mark.parametrize("m, n, k", [(4000, 3072, 256), (2080, 1024, 320)])
def test_matmul_pair_kernel_ragged_rows(m, n, k, rng):
    """More 256-row tiles than CTA pairs, M not a multiple of the tile nor of the 32-row store boxes: the CTA-pair
    kernel with its staged bulk stores, bias + GELU + residual in the epilogue; the tensor map clips the last rows."""
    dtype = torch.float16
    a, w = rng.standard_normal((m, k)).astype(np.float32), (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    bias, res = rng.standard_normal(n).astype(np.float32), rng.standard_normal((m, n)).astype(np.float32)
    guard = torch.full((m + 64, n), 7.0, dtype=dtype, device="cuda")
    y = guard[:m]
    donnx.ONNXFusedMatMul(A=dev(a, dtype), B=dev(w, dtype), Bias=dev(bias, dtype), Residual=dev(res, dtype), Y=y, transB=1,
                          activation="Gelu")
    pre = ops.matmul(rounded(a, dtype), rounded(w, dtype).T.copy()) + rounded(bias, dtype)
    ref = ops.gelu_chain(pre.astype(np.float32)) + rounded(res, dtype)
    assert_close(y, ref, dtype, what=f"pair gemm {m}x{n}x{k}")
    assert bool((guard[m:] == 7.0).all()), "rows past M were written"
    status_ok()


@pytest.mark.parametrize("m, n, k", [(1000, 200, 360), (4096, 120, 784), (300, 256, 1024), (2048, 128, 288), (4096, 100, 2048), (640, 128, 4096),
                                     (8192, 64, 516)])
def test_gemm_fp32_tensor_core_path(m, n, k, rng):
    """fp32 Gemm(transB=1) large enough for the three-pass TF32 tensor-core kernel: ragged M, N and K, bias + ReLU;
    few output tiles (K split over clusters of 2 or 4 CTAs, also with a share of K that is empty) and many.
    The result must meet the fp32 tolerance (rtol 1e-4), which a single TF32 pass would not."""
    a, w, c = (rng.standard_normal((m, k)).astype(np.float32), (rng.standard_normal((n, k)) * 0.1).astype(np.float32),
               rng.standard_normal(n).astype(np.float32))
    ref = np.maximum(a.astype(np.float64) @ w.astype(np.float64).T + c, 0.0)
    y = empty((m, n), torch.float32)
    donnx.ONNXFusedMatMul(A=dev(a), B=dev(w), Bias=dev(c), Y=y, transB=1, activation="Relu")
    # sums of K products cancel down to values near zero, so the operator tolerance gets the absolute floor of an
    # fp32 dot product of this length ...
    assert_close(y, ref, torch.float32, atol=3e-5, what=f"fp32 gemm {m}x{n}x{k}")
    # ... and the forward error is checked against what it scales with: |error| <= 2e-6 * sum_k |a_ik| |w_jk|
    # (the split keeps about 21 bits of each operand; a single TF32 pass would sit near 5e-4)
    scale = np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64).T + np.abs(c)
    ratio = (np.abs(y.cpu().numpy().astype(np.float64) - ref) / scale).max()
    print(f"3xTF32 {m}x{n}x{k}: forward error {ratio:.2e} of sum |a||w|, max abs {np.abs(y.cpu().numpy() - ref).max():.2e}")
    assert ratio < 2e-6, f"3xTF32 forward error {ratio:.2e} of sum |a||w|"
    status_ok()


@pytest.mark.parametrize("m, n, k", [(512, 520, 384), (1024, 256, 260), (4096, 1024, 1024), (777, 132, 1000)])
def test_matmul_fp32_tensor_core_path_with_b_in_onnx_layout(m, n, k, rng):
    """fp32 MatMul with B as ONNX gives it ([K, N], N contiguous) on the same three-pass TF32 kernel (B read as the
    MN-major operand): ragged M, N and K; one split launch and one product."""
    if os.environ.get("B200ML_TF32X3", "1") == "0":
        pytest.skip("the fp32 tensor-core GEMM is switched off")
    a, b = rng.standard_normal((m, k)).astype(np.float32), (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    guard = torch.full((m * n + 4096, ), 7.0, dtype=torch.float32, device="cuda")
    y = guard[:m * n].view(m, n)
    before = L.launch_count()
    donnx.ONNXMatMul(A=dev(a), B=dev(b), Y=y)
    assert L.launch_count() - before == 2, "expected the operand split and the tensor-core product"
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    ratio = (np.abs(y.cpu().numpy().astype(np.float64) - ref) / scale).max()
    assert ratio < 2e-6, f"3xTF32 forward error {ratio:.2e} of sum |a||b|"
    assert_close(y, ops.matmul(a, b), torch.float32, atol=3e-5, what=f"fp32 matmul {m}x{n}x{k}")
    assert bool((guard[m * n:] == 7.0).all()), "written past the end of Y"
    status_ok()


def test_gemm_golden_and_rules():
    g = gold("gemm")
    y = empty((7, 5), torch.float32)
    donnx.ONNXGemm(A=dev(g["a"]), B=dev(g["b"]), C=dev(g["c"]), Y=y, alpha=0.5, beta=2.0, transB=1)
    assert_close(y, g["y"], what="gemm alpha/beta/transB")
    donnx.ONNXGemm(A=dev(g["at"]), B=dev(g["bt"]), C=dev(g["c2"]), Y=y, transA=1)
    assert_close(y, g["y2"], what="gemm transA, full C")
    status_ok()


@pytest.mark.parametrize("dtype", DTYPES)
def test_gemm_linear_export(dtype, rng):
    """nn.Linear as exported: Gemm(alpha=1, beta=1, transB=1) with C[N]."""
    a, w, c = (rng.standard_normal((512, 784)).astype(np.float32), rng.standard_normal((120, 784)).astype(np.float32) * 0.05,
               rng.standard_normal(120).astype(np.float32))
    ref = ops.gemm(rounded(a, dtype), rounded(w, dtype), rounded(c, dtype), trans_b=1)
    y = empty((512, 120), dtype)
    donnx.ONNXGemm(A=dev(a, dtype), B=dev(w, dtype), C=dev(c, dtype), Y=y, transB=1)
    assert_close(y, ref, dtype, what="gemm linear")


@pytest.mark.parametrize("m, n, k", [(4096, 32, 120), (4096, 10, 32), (300, 1, 4), (257, 17, 64), (1000, 24, 300), (512, 8, 8)])
@pytest.mark.parametrize("trans_b", [0, 1])
def test_gemm_skinny_outputs(m, n, k, trans_b, rng):
    """fp32 products with few output columns (classifier heads, the last layers of the MLP; up to 16 columns take the
    kernel that keeps all of B in shared memory): bias, ReLU and both weight layouts, against the oracle in fp64 terms."""
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k) if trans_b else (k, n)) * 0.1).astype(np.float32)
    c = rng.standard_normal(n).astype(np.float32)
    ref = ops.gemm(a, w, c, trans_b=trans_b, acc_dtype=np.float64)
    y = empty((m, n), torch.float32)
    donnx.ONNXGemm(A=dev(a), B=dev(w), C=dev(c), Y=y, transB=trans_b)
    assert_close(y, ref, what=f"skinny gemm {m}x{n}x{k}")
    yr = empty((m, n), torch.float32)
    K.gemm(dev(a), dev(w), yr, b_layout=trans_b, bias=dev(c), act=L.EPI_RELU, residual=y, alpha=0.5)
    want = np.maximum(0.5 * (a.astype(np.float64) @ (w.T if trans_b else w).astype(np.float64)) + c, 0.0) + y.cpu().numpy()
    assert_close(yr, want.astype(np.float32), what="skinny gemm with bias, ReLU, residual")
    status_ok()


def test_einsum_reference_test():
    """tests/pure_expansions/test_expansions.py:387-405 ('bij, jk -> bik')."""
    g = gold("einsum")
    y = empty(g["y"].shape, torch.float32)
    donnx.ONNXEinsum(Inputs__0=dev(g["a"]), Inputs__1=dev(g["b"]), Output=y, equation="bij, jk -> bik")
    assert_close(y, g["y"], what="einsum bij,jk->bik")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("eq, shapes", [("bik,bjk->bij", [(4, 160, 64), (4, 96, 64)]), ("ki,kj->ij", [(64, 40), (64, 24)]),
                                        ("abcd->acbd", [(2, 3, 4, 5)]), ("yzik,yzkj->yzij", [(2, 3, 16, 8), (2, 3, 8, 24)])])
def test_einsum_forms(dtype, eq, shapes, rng):
    arrs = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    ref = ops.einsum(eq, *[rounded(a, dtype) for a in arrs])
    y = empty(ref.shape, dtype)
    kwargs = {"Inputs__%d" % i: dev(a, dtype) for i, a in enumerate(arrs)}
    donnx.ONNXEinsum(Output=y, equation=eq, **kwargs)
    assert_close(y, ref, dtype, what=eq)


# ------------------------------------------------------------------------------------------------
# Softmax / reductions / element-wise
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_softmax_golden_axes(dtype):
    g = gold("softmax")
    x = g["x"]
    for axis, key in ((3, "softmax_axis3"), (1, "softmax_axis1"), (-1, "softmax_axis3")):
        y = empty(x.shape, dtype)
        donnx.ONNXSoftmax(input=dev(x, dtype), output=y, axis=axis)
        ref = ops.softmax(rounded(x, dtype), axis)
        assert_close(y, ref, dtype, what=f"softmax axis {axis}")
        if dtype == torch.float32:
            assert_close(y, g[key], dtype, what=f"softmax golden axis {axis}")
    y = empty((5, 16), dtype)
    donnx.ONNXLogSoftmax(input=dev(x[0, 0], dtype), output=y, axis=1)
    assert_close(y, ops.log_softmax(rounded(x[0, 0], dtype), 1), dtype, atol=1e-2 if dtype == torch.float16 else None,
                 what="logsoftmax")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape, axis", [((4, 16, 64, 512), 3), ((4096, 10), 1), ((3, 1), 1), ((2, 5000), 1), ((7, 333), 1), ((1, 1, 1, 8), 3)])
def test_softmax_shapes(dtype, shape, axis, rng):
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    y = empty(shape, dtype)
    donnx.ONNXSoftmax(input=dev(x, dtype), output=y, axis=axis)
    assert_close(y, ops.softmax(rounded(x, dtype), axis), dtype, what=f"softmax {shape}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, cols", [(4096, 10), (37, 3), (5, 100), (33, 255), (9, 17), (64, 2)])
def test_softmax_short_rows_with_scale_mask_and_log(dtype, rows, cols, rng):
    """Rows the packet kernels cannot take (classifier heads): several lanes per row, several rows per warp."""
    x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
    m = (rng.standard_normal((rows, cols)) * 2).astype(np.float32)
    xd, md = dev(x, dtype), dev(m, dtype)
    xr, mr = rounded(x, dtype), rounded(m, dtype)
    y = empty((rows, cols), dtype)
    K.softmax(xd, y, rows=rows, cols=cols, scale=0.5, mask=md)
    assert_close(y, ops.softmax(xr * np.float32(0.5) + mr, 1), dtype, what="short softmax with scale and mask")
    K.softmax(xd, y, rows=rows, cols=cols, log=True)
    assert_close(y, ops.log_softmax(xr, 1), dtype, atol=1e-2 if dtype == torch.float16 else None, what="short log-softmax")
    status_ok()


@pytest.mark.parametrize("kind, keep, axes", [("Sum", True, [0]), ("Sum", False, [-1]), ("Sum", True, [0, -1]), ("Max", False, [0, -1]),
                                              ("Max", True, [0]), ("Max", True, [-1]), ("Mean", True, [-1]), ("Mean", True, [0, -1]),
                                              ("Mean", False, [0]), ("Min", True, [1])])
def test_reduce_reference_cases(kind, keep, axes):
    """tests/pure_expansions/test_expansions.py:187-237."""
    g = gold("reduce")
    key = "%s_%d_%s" % (kind.lower(), int(keep), "_".join(str(a) for a in axes))
    y = empty(g[key].shape, torch.float32)
    getattr(donnx, "ONNXReduce" + kind)(data=dev(g["x"]), reduced=y, axes=axes, keepdims=int(keep))
    assert_close(y, g[key], atol=1e-5, what=key)


def test_reduce_to_scalar_and_long_rows(rng):
    g = gold("reduce")
    y = empty((), torch.float32)
    donnx.ONNXReduceMean(data=dev(g["x"]), reduced=y, keepdims=0)  # test_expansions.py:240-278
    assert_close(y, g["mean_scalar"], what="mean to scalar")
    big = rng.standard_normal((2, 1_500_000)).astype(np.float32)
    y = empty((2, ), torch.float32)
    donnx.ONNXReduceSum(data=dev(big), reduced=y, axes=[1], keepdims=0)  # sliced rows through the scratch buffer
    assert_close(y, big.astype(np.float64).sum(1), rtol=1e-4, atol=1e-2, what="long-row sum")
    one = rng.standard_normal((3_000_000, )).astype(np.float32)
    y = empty((), torch.float32)
    donnx.ONNXReduceMax(data=dev(one), reduced=y, keepdims=0)
    assert float(y) == float(one.max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_elementwise_golden(dtype):
    g = gold("elementwise")
    x, yv = g["x"], g["y"]
    xd, yd = dev(x, dtype), dev(yv, dtype)
    xr, yr = rounded(x, dtype), rounded(yv, dtype)
    out = empty(x.shape, dtype)
    for node, ref in ((donnx.ONNXAdd, ops.add(xr, yr)), (donnx.ONNXSub, ops.sub(xr, yr)), (donnx.ONNXMul, ops.mul(xr, yr)),
                      (donnx.ONNXDiv, ops.div(xr, yr))):
        node(A=xd, B=yd, C=out)
        assert_close(out, ref, dtype, what=node.__name__)
    donnx.ONNXPow(X=xd, Y=torch.tensor(2.0, dtype=dtype, device="cuda"), Z=out)
    assert_close(out, ops.pow_(xr, np.float32(2.0)), dtype, what="pow")
    for node, conn, ref in ((donnx.ONNXErf, ("input", "output"), ops.erf(xr)), (donnx.ONNXTanh, ("input", "output"), ops.tanh(xr)),
                            (donnx.ONNXExp, ("input", "output"), ops.exp(xr)), (donnx.ONNXRelu, ("X", "Y"), ops.relu(xr)),
                            (donnx.ONNXSigmoid, ("X", "Y"), ops.sigmoid(xr)), (donnx.ONNXSoftplus, ("X", "Y"), ops.softplus(xr)),
                            (donnx.ONNXGelu, ("X", "Y"), ops.gelu_chain(xr)), (donnx.ONNXSwish, ("X", "Y"), ops.swish(xr)),
                            (donnx.ONNXIdentity, ("input", "output"), xr)):
        node(**{conn[0]: xd, conn[1]: out})
        assert_close(out, ref, dtype, what=node.__name__)
    donnx.ONNXLeakyRelu(X=xd, Y=out, alpha=0.1)
    assert_close(out, ops.leaky_relu(xr, 0.1), dtype, what="leakyrelu")
    donnx.ONNXSqrt(X=dev(np.abs(x), dtype), Y=out)
    assert_close(out, ops.sqrt(np.abs(xr)), dtype, what="sqrt")


@pytest.mark.parametrize("dtype", DTYPES)
def test_broadcast_forms(dtype, rng):
    a = rng.standard_normal((8, 1, 16, 24)).astype(np.float32)
    b = rng.standard_normal((1, 5, 16, 1)).astype(np.float32)
    out = empty((8, 5, 16, 24), dtype)
    donnx.ONNXAdd(A=dev(a, dtype), B=dev(b, dtype), C=out)
    assert_close(out, ops.add(rounded(a, dtype), rounded(b, dtype)), dtype, what="general broadcast")
    x = rng.standard_normal((4, 7, 1024)).astype(np.float32)
    bias = rng.standard_normal((1024, )).astype(np.float32)
    out = empty(x.shape, dtype)
    donnx.ONNXSub(A=dev(bias, dtype), B=dev(x, dtype), C=out)
    assert_close(out, ops.sub(rounded(bias, dtype), rounded(x, dtype)), dtype, what="vector - tensor")
    mean = x.mean(-1, keepdims=True).astype(np.float32)
    donnx.ONNXSub(A=dev(x, dtype), B=dev(mean, dtype), C=out)
    assert_close(out, ops.sub(rounded(x, dtype), rounded(mean, dtype)), dtype, what="row broadcast")


def test_cast_roundtrip(rng):
    x = rng.standard_normal((1000, 33)).astype(np.float32)
    h = empty(x.shape, torch.float16)
    donnx.ONNXCast(input=dev(x), output=h, to=10)
    assert torch.equal(h.cpu(), torch.from_numpy(x).half())
    f = empty(x.shape, torch.float32)
    donnx.ONNXCast(input=h, output=f, to=1)
    assert torch.equal(f.cpu(), torch.from_numpy(x).half().float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape, perm", [((8, 64, 16, 64), (0, 2, 1, 3)), ((2, 40, 4, 64), (0, 2, 3, 1)), ((1024, 1000), (1, 0)),
                                         ((3, 5, 7), None), ((2, 3, 4, 5, 6), (4, 0, 3, 1, 2)), ((17, ), (0, ))])
def test_transpose_bit_exact(dtype, shape, perm, rng):
    x = rng.standard_normal(shape).astype(np.float32)
    xd = dev(x, dtype)
    ref = ops.transpose(xd.cpu().numpy(), perm)
    y = empty(ref.shape, dtype)
    donnx.ONNXTranspose(data=xd, transposed=y, **({} if perm is None else {"perm": list(perm)}))
    assert np.array_equal(y.cpu().numpy(), ref)


def test_reshape_like_nodes(rng):
    x = rng.standard_normal((4, 6, 10)).astype(np.float32)
    y = empty((24, 10), torch.float32)
    donnx.ONNXReshape(data=dev(x), reshaped=y)
    assert np.array_equal(y.cpu().numpy(), x.reshape(24, 10))
    y = empty((4, 60), torch.float32)
    donnx.ONNXFlatten(input=dev(x), output=y, axis=1)
    assert np.array_equal(y.cpu().numpy(), ops.flatten(x, 1))


@pytest.mark.parametrize("dtype", DTYPES)
def test_layernorm_fused_matches_chain(dtype):
    g = gold("layernorm")
    x, ga, be = g["x"], g["gamma"], g["beta"]
    y = empty(x.shape, dtype)
    donnx.ONNXLayerNormalization(X=dev(x, dtype), Scale=dev(ga, dtype), B=dev(be, dtype), Y=y, epsilon=1e-12)
    assert_close(y, ops.layernorm_chain(rounded(x, dtype), rounded(ga, dtype), rounded(be, dtype), 1e-12), dtype, what="layernorm")
    r = np.roll(x, 1, axis=0)
    donnx.ONNXLayerNormalization(X=dev(x, dtype), Residual=dev(r, dtype), Scale=dev(ga, dtype), B=dev(be, dtype), Y=y, epsilon=1e-12)
    ref = ops.layernorm_chain(rounded(x, dtype) + rounded(r, dtype), rounded(ga, dtype), rounded(be, dtype), 1e-12)
    assert_close(y, ref, dtype, what="layernorm + residual")


@pytest.mark.parametrize("m, n, k", [(4096, 1024, 1024), (300, 512, 264), (128, 256, 64), (1000, 1024, 4096)])
@pytest.mark.parametrize("trans_b", [1, 0])
def test_matmul_with_layernorm_epilogue(m, n, k, trans_b, rng):
    """FusedMatMul with LnScale / LnBias: bias + residual + LayerNorm inside the GEMM (cluster-wide row statistics)."""
    dtype = torch.float16
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k) if trans_b else (k, n)) * 0.05).astype(np.float32)
    bias, res = rng.standard_normal(n).astype(np.float32), rng.standard_normal((m, n)).astype(np.float32)
    gamma, beta = (1 + 0.2 * rng.standard_normal(n)).astype(np.float32), (0.2 * rng.standard_normal(n)).astype(np.float32)
    y = empty((m, n), dtype)
    donnx.ONNXFusedMatMul(A=dev(a, dtype), B=dev(w, dtype), Bias=dev(bias, dtype), Residual=dev(res, dtype), LnScale=dev(gamma, dtype),
                          LnBias=dev(beta, dtype), Y=y, transB=trans_b, ln_epsilon=1e-12)
    wr = rounded(w, dtype)
    pre = ops.matmul(rounded(a, dtype), wr.T.copy() if trans_b else wr) + rounded(bias, dtype) + rounded(res, dtype)
    ref = ops.layernorm_chain(pre.astype(np.float32), rounded(gamma, dtype), rounded(beta, dtype), 1e-12)
    assert_close(y, ref, dtype, atol=5e-3, what=f"gemm+layernorm {m}x{n}x{k}")
    status_ok()


def test_matmul_with_layernorm_split_path(rng):
    """A width the fused kernel does not cover (N = 384) runs as GEMM + LayerNorm and gives the same answer."""
    dtype = torch.float16
    m, n, k = 200, 384, 128
    a, w = rng.standard_normal((m, k)).astype(np.float32), (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    gamma = (1 + 0.2 * rng.standard_normal(n)).astype(np.float32)
    y = empty((m, n), dtype)
    donnx.ONNXFusedMatMul(A=dev(a, dtype), B=dev(w, dtype), LnScale=dev(gamma, dtype), Y=y, transB=1, ln_epsilon=1e-5)
    pre = ops.matmul(rounded(a, dtype), rounded(w, dtype).T.copy())
    ref = ops.layernorm_chain(pre.astype(np.float16).astype(np.float32), rounded(gamma, dtype), np.zeros(n, np.float32), 1e-5)
    assert_close(y, ref, dtype, atol=5e-3, what="gemm then layernorm")


# ------------------------------------------------------------------------------------------------
# Conv
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("idx, bias", [(0, True), (1, False), (2, True), (3, False)])
def test_conv_simple_reference_test(idx, bias):
    """tests/pure_expansions/test_conv_expansion.py:9-66 through the traced-program frontend."""
    g = gold("conv")
    X, W, Z = g["x%d" % idx], g["w%d" % idx], g["y%d" % idx]
    dace_Z = np.zeros_like(Z)
    if bias:
        B = g["b%d" % idx]

        @donnx.program
        def conv(X_: (np.float32, X.shape), W_: (np.float32, W.shape), B_: (np.float32, B.shape), Z_: (np.float32, Z.shape)):
            donnx.ONNXConv(X=X_, W=W_, B=B_, Y=Z_)

        sdfg = conv.to_sdfg()
        sdfg.expand_library_nodes()
        sdfg(X_=X, W_=W, Z_=dace_Z, B_=B)
    else:

        @donnx.program
        def conv(X_: (np.float32, X.shape), W_: (np.float32, W.shape), Z_: (np.float32, Z.shape)):
            donnx.ONNXConv(X=X_, W=W_, Y=Z_)

        sdfg = conv.to_sdfg()
        sdfg.expand_library_nodes()
        sdfg(X_=X, W_=W, Z_=dace_Z)
    assert np.allclose(Z, dace_Z)
    assert_close(dace_Z, Z, torch.float32, what="conv golden")


def test_conv_strided_padded_grouped_golden():
    g = gold("conv")
    y = empty(g["ys"].shape, torch.float32)
    donnx.ONNXConv(X=dev(g["xs"]), W=dev(g["ws"]), Y=y, strides=[2, 2])
    assert_close(y, g["ys"], what="strided conv")
    y = empty(g["yg"].shape, torch.float32)
    donnx.ONNXConv(X=dev(g["xg"]), W=dev(g["wg"]), B=dev(g["bg"]), Y=y, strides=[2, 1], pads=[1, 0, 2, 1], dilations=[1, 2], group=2)
    assert_close(y, g["yg"], what="strided / padded / dilated / grouped conv")
    y = empty(g["yd"].shape, torch.float32)
    donnx.ONNXConv(X=dev(g["xd"]), W=dev(g["wd"]), Y=y, pads=[1, 1, 1, 1], group=12)
    assert_close(y, g["yd"], what="depthwise conv")
    p = empty((2, 12, 1, 1), torch.float32)
    donnx.ONNXGlobalAveragePool(X=dev(g["xd"]), Y=p)
    assert_close(p, g["gap"], what="global average pool")
    status_ok()


def test_conv_config1_full_size(rng):
    """BASELINE config 1: X[32,3,64,64] ~ N(0,1), W[16,3,3,3] ~ U(0,1), stride 2, no pad, no bias."""
    x = rng.standard_normal((32, 3, 64, 64)).astype(np.float32)
    w = rng.random((16, 3, 3, 3), np.float32)
    y = empty((32, 16, 31, 31), torch.float32)
    donnx.ONNXConv(X=dev(x), W=dev(w), Y=y, strides=[2, 2])
    assert_close(y, ops.conv2d(x, w, strides=(2, 2)), what="config 1")


@pytest.mark.parametrize("cin, cout, hw", [(24, 144, (56, 56)), (144, 24, (56, 56)), (5, 40, (6, 10)), (40, 7, (4, 4)), (3, 3, (5, 5))])
def test_conv_pointwise(cin, cout, hw, rng):
    x = rng.standard_normal((3, cin) + hw).astype(np.float32)
    w = (rng.standard_normal((cout, cin, 1, 1)) * 0.1).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    y = empty((3, cout) + hw, torch.float32)
    donnx.ONNXConv(X=dev(x), W=dev(w), B=dev(b), Y=y)
    assert_close(y, ops.conv2d(x, w, b), what=f"1x1 conv {cin}->{cout}")


@pytest.mark.parametrize("n, cin, cout, hw", [(8, 24, 144, (56, 56)), (8, 144, 24, (56, 56)), (16, 40, 100, (36, 36)), (4, 100, 40, (64, 64)),
                                              (3, 8, 8, (150, 152)), (24, 24, 256, (28, 28)), (6, 31, 9, (64, 60)), (6, 32, 64, (64, 60)), (2, 33, 17, (128, 64)), (16, 72, 72, (30, 40))])
@pytest.mark.parametrize("act", ["", "Swish", "Relu"])
def test_conv_pointwise_tensor_core(n, cin, cout, hw, act, rng):
    """1x1 convolutions large enough for the tensor-core kernel (3 x TF32, NCHW operand read MN-major through TMA):
    ragged last pixel tile (H * W not a multiple of 128), channel counts that are not whole 32- or 16-blocks,
    squeeze-excite gate on the input, bias, activation and residual add.  Against the oracle at the fp32 tolerance,
    and against a float64 product at a bound that a single-TF32 product (relative error 5e-4) would break."""
    if os.environ.get("B200ML_CONV_TC", "1") == "0":
        pytest.skip("the tensor-core convolution is switched off")
    x = rng.standard_normal((n, cin) + hw).astype(np.float32)
    w = (rng.standard_normal((cout, cin, 1, 1)) * 0.1).astype(np.float32)
    b = (rng.standard_normal(cout) * 3).astype(np.float32)
    gate = rng.random((n, cin, 1, 1)).astype(np.float32)
    res = rng.standard_normal((n, cout) + hw).astype(np.float32)
    guard = torch.full((n * cout * hw[0] * hw[1] + 4096, ), 7.0, dtype=torch.float32, device="cuda")
    y = guard[:n * cout * hw[0] * hw[1]].view((n, cout) + hw)
    before = L.launch_count()
    donnx.ONNXFusedConv(X=dev(x), W=dev(w), B=dev(b), Gate=dev(gate), Residual=dev(res), Y=y, activation=act)
    assert L.launch_count() - before == 2, "expected the weight split and the tensor-core kernel"
    xg = x.astype(np.float64) * gate.astype(np.float64)
    pre = np.einsum("mc,nchw->nmhw", w[:, :, 0, 0].astype(np.float64), xg) + b.astype(np.float64)[None, :, None, None]
    post = {"": pre, "Swish": pre / (1 + np.exp(-pre)), "Relu": np.maximum(pre, 0)}[act] + res
    mag = np.einsum("mc,nchw->nmhw", np.abs(w[:, :, 0, 0]).astype(np.float64), np.abs(xg)) + np.abs(b)[None, :, None, None] + np.abs(res)
    err = np.abs(y.double().cpu().numpy() - post)
    assert (err <= 4e-6 * mag + 1e-6).all(), "3 x TF32 accuracy lost: worst error / magnitude %.3g" % float((err / (mag + 1e-9)).max())
    oracle = ops.conv2d((x * gate).astype(np.float32), w, b)
    oracle = {"": oracle, "Swish": ops.swish(oracle), "Relu": ops.relu(oracle)}[act] + res
    assert_close(y, oracle, what=f"1x1 conv {cin}->{cout} {hw} {act}", atol=2e-5)
    assert bool((guard[n * cout * hw[0] * hw[1]:] == 7.0).all()), "written past the end of Y"
    status_ok()


@pytest.mark.parametrize("n, cin, cout, hw, k, pads", [(8, 16, 32, (48, 48), (3, 3), (1, 1, 1, 1)), (4, 64, 64, (56, 56), (3, 3), (1, 1, 1, 1)),
                                                       (6, 10, 40, (36, 40), (5, 5), (2, 2, 2, 2)), (4, 24, 200, (30, 44), (3, 3), (0, 1, 0, 1)),
                                                       (3, 32, 16, (80, 96), (3, 5), (1, 2, 1, 2)), (5, 12, 48, (40, 64), (3, 3), (2, 0, 0, 2)),
                                                       (2, 8, 32, (64, 64), (7, 7), (3, 3, 3, 3)), (64, 128, 128, (16, 16), (3, 3), (1, 1, 1, 1)),
                                                       (24, 32, 48, (14, 14), (3, 3), (1, 1, 1, 1)), (96, 16, 32, (7, 7), (3, 3), (1, 1, 1, 1)),
                                                       (10, 8, 24, (30, 27), (3, 3), (1, 1, 1, 1)), (6, 8, 16, (32, 32), (3, 3), (0, 0, 0, 0)),
                                                       (8, 9, 40, (21, 37), (5, 3), (2, 1, 2, 1)), (32, 16, 24, (20, 18), (3, 3), (0, 0, 0, 0)),
                                                       (40, 8, 20, (12, 12), (5, 5), (2, 2, 2, 2)), (16, 24, 136, (33, 9), (3, 3), (1, 1, 1, 1)),
                                                       (16, 16, 32, (24, 20), (3, 3), (1, 1, 1, 1)), (12, 8, 16, (20, 24), (3, 3), (0, 0, 0, 0)),
                                                       (8, 32, 64, (56, 56), (3, 3), (1, 1, 1, 1, 2, 2)), (24, 16, 32, (30, 30), (3, 3), (0, 0, 0, 0, 2, 2)),
                                                       (6, 16, 24, (40, 48), (3, 3), (1, 1, 1, 1, 2, 1)), (8, 64, 96, (48, 64), (1, 1), (0, 0, 0, 0, 2, 2)),
                                                       (8, 12, 20, (41, 52), (5, 5), (2, 2, 2, 2, 1, 2)), (6, 8, 16, (64, 64), (5, 5), (2, 2, 2, 2, 2, 2))])
@pytest.mark.parametrize("act", ["", "Relu"])
def test_conv_kxk_tensor_core(n, cin, cout, hw, k, pads, act, rng):
    """k x k stride-1 convolutions large enough for the implicit-GEMM kernel (3 x TF32; kernel columns as shifted copies
    of the input window, kernel rows as descriptor offsets): ragged tiles in both directions, channel counts that are
    not whole 8- or 32-blocks, more than one block of output channels, asymmetric padding, non-square kernels, bias,
    activation and residual, strides of 2 (also mixed, and a strided 1x1); image widths that are not a multiple of 4 (no tensor map for X and Y: the warps load and
    store themselves), narrow images (two image rows per operand line).  Against the oracle at the fp32 tolerance, and against a float64 convolution at a bound
    that a single-TF32 product (relative error 5e-4) would break."""
    if os.environ.get("B200ML_CONV_TC", "1") == "0":
        pytest.skip("the tensor-core convolution is switched off")
    strides = tuple(pads[4:]) or (1, 1)  # a six-entry pads tuple carries the strides behind the four pads
    pads = tuple(pads[:4])
    x = rng.standard_normal((n, cin) + hw).astype(np.float32)
    w = (rng.standard_normal((cout, cin) + k) * 0.1).astype(np.float32)
    b = (rng.standard_normal(cout) * 3).astype(np.float32)
    oracle = ops.conv2d(x, w, b, strides=strides, pads=pads)
    res = rng.standard_normal(oracle.shape).astype(np.float32)
    guard = torch.full((oracle.size + 4096, ), 7.0, dtype=torch.float32, device="cuda")
    y = guard[:oracle.size].view(oracle.shape)
    before = L.launch_count()
    donnx.ONNXFusedConv(X=dev(x), W=dev(w), B=dev(b), Residual=dev(res), Y=y, pads=list(pads), strides=list(strides), activation=act)
    assert L.launch_count() - before == 2, "expected the weight split and the implicit-GEMM kernel"
    pt, pl, pb, pr = pads
    xp = torch.nn.functional.pad(torch.from_numpy(x).double(), (pl, pr, pt, pb))
    pre = torch.nn.functional.conv2d(xp, torch.from_numpy(w).double(), torch.from_numpy(b).double(), stride=strides).numpy()
    mag = torch.nn.functional.conv2d(xp.abs(), torch.from_numpy(w).double().abs(), torch.from_numpy(b).double().abs(), stride=strides).numpy() + np.abs(res)
    post = {"": pre, "Relu": np.maximum(pre, 0)}[act] + res
    err = np.abs(y.double().cpu().numpy() - post)
    assert (err <= 4e-6 * mag + 1e-6).all(), "3 x TF32 accuracy lost: worst error / magnitude %.3g" % float((err / (mag + 1e-9)).max())
    # the oracle adds its cin * kh * kw terms one after the other in fp32: its own rounding error grows with the terms'
    # magnitudes, so they enter the bound next to the fp32 tolerance
    oracle = {"": oracle, "Relu": ops.relu(oracle)}[act] + res
    err_o = np.abs(y.cpu().numpy().astype(np.float64) - oracle)
    bad = err_o > 2e-5 + 1e-4 * np.abs(oracle) + 4e-6 * mag
    assert not bad.any(), f"{k} conv {cin}->{cout} {hw} {pads} {act}: {bad.sum()} of {bad.size} elements away from the oracle, worst {err_o.max():.3g}"
    assert bool((guard[oracle.size:] == 7.0).all()), "written past the end of Y"
    status_ok()


@pytest.mark.parametrize("c, hw, pads", [(144, (56, 56), (1, 1, 1, 1)), (5, (7, 8), (1, 1, 1, 1)), (3, (13, 12), (1, 1, 1, 1)), (6, (33, 64), (1, 1, 1, 1)),
                                         (4, (1, 16), (1, 1, 1, 1)), (5, (9, 10), (1, 1, 1, 1)), (4, (12, 12), (0, 1, 1, 0)), (2, (70, 72), (1, 1, 1, 1))])
@pytest.mark.parametrize("act", ["", "Swish"])
def test_depthwise_3x3_forms(c, hw, pads, act, rng):
    """Depthwise 3x3 on the four-columns-per-lane kernel (pad 1, width a multiple of 4 up to 64), on the
    column-per-lane kernel (other widths and pads) and on the staged kernel (wide planes), with the pooled mean."""
    x = rng.standard_normal((3, c) + hw).astype(np.float32)
    w = (rng.standard_normal((c, 1, 3, 3)) * 0.3).astype(np.float32)
    b = rng.standard_normal(c).astype(np.float32)
    ref = ops.conv2d(x, w, b, pads=pads, group=c)
    if act:
        ref = ops.swish(ref)
    y = empty(ref.shape, torch.float32)
    pool = empty((3, c, 1, 1), torch.float32)
    donnx.ONNXFusedConv(X=dev(x), W=dev(w), B=dev(b), Y=y, Pool=pool, pads=list(pads), group=c, activation=act)
    assert_close(y, ref, what=f"depthwise {hw} {pads} {act}", atol=2e-5)
    assert_close(pool, ref.mean(axis=(2, 3), keepdims=True), what="pooled mean", atol=2e-5)
    status_ok()


# ------------------------------------------------------------------------------------------------
# Edge cases of the C ABI
# ------------------------------------------------------------------------------------------------
def test_empty_tensors_launch_nothing():
    before = L.launch_count()
    x = empty((0, 16), torch.float32)
    K.unary(x, x, L.UN_RELU)
    K.softmax(x, x, rows=0, cols=16)
    K.gemm(empty((0, 8), torch.float16), empty((8, 4), torch.float16), empty((0, 4), torch.float16))
    assert L.launch_count() == before


def test_invalid_arguments_raise():
    a, b = empty((4, 8), torch.float16), empty((9, 4), torch.float16)
    with pytest.raises(L.B200Error):
        K.gemm(a, b, empty((4, 4), torch.float16))
    with pytest.raises(L.B200Error):
        K.unary(torch.zeros(4), torch.zeros(4), L.UN_RELU)  # CPU tensors: no CPU path
    with pytest.raises(L.Unsupported):
        K.unary(empty((4, ), torch.float64), empty((4, ), torch.float64), L.UN_RELU)


# ------------------------------------------------------------------------------------------------
# Every case of tests/golden/ref_pure_expansions.*: vectors computed by the reference's own source
# (pure_implementations.py / img_op_implementations.py executed under numpy) against the CUDA path
# ------------------------------------------------------------------------------------------------
import ref_cases  # noqa: E402


@pytest.mark.parametrize("case", ref_cases.REF_CASES, ids=[c["case"] for c in ref_cases.REF_CASES])
def test_kernels_match_reference_source(case):
    results = ref_cases.frontend_outputs(case, ref_cases.ref_arrays(), donnx, torch)
    for conn, (got, want) in results.items():
        assert got.shape == want.shape and got.dtype == want.dtype, (conn, got.shape, want.shape, got.dtype, want.dtype)
        if case["op"] in ref_cases.BIT_EXACT_OPS or not np.issubdtype(want.dtype, np.floating):
            assert np.array_equal(got, want), f"{case['case']}:{conn} is not bit-exact"
        else:
            assert_close(got, want, torch.float32, what=f"{case['case']}:{conn}")
    status_ok()


@pytest.mark.parametrize("name", ["conv_igemm_c4_k5_f16", "conv_igemm_c8_k3_f16", "conv_pointwise_tc"])
def test_tensor_core_convolutions_match_the_reference_loop_nest(name):
    """The fixtures produced by the reference's own ``PureConv2D`` loop nest (``img_op_implementations.py:217-288``,
    executed as Python) at sizes the implicit-GEMM kernel and the 1x1 kernel take: the tensor-core path did run (weight
    split + kernel), and agrees at the fp32 tolerance."""
    if os.environ.get("B200ML_CONV_TC", "1") == "0":
        pytest.skip("the tensor-core convolution is switched off")
    case = next(c for c in ref_cases.REF_CASES if c["case"] == name)
    before = L.launch_count()
    results = ref_cases.frontend_outputs(case, ref_cases.ref_arrays(), donnx, torch)
    assert L.launch_count() - before == 2, "expected the weight split and the tensor-core kernel"
    got, want = results["Y"]
    assert_close(got, want, torch.float32, what=name)
    status_ok()


def test_python_implementations_through_the_helper_api(rng):
    """An implementation written with ``python_pure_op_implementation`` (a function over the connectors' tensors) and one
    that returns a nested SDFG built with ``empty_sdfg_for_node`` (Softplus as Exp -> Add 1 -> Log from this library's own
    nodes), selected per node, against the oracle."""
    from daceml_b200 import sdfg as sd
    from daceml_b200.onnx.forward_implementation_abc import ONNXForward
    from daceml_b200.onnx.op_implementations.utils import empty_sdfg_for_node, op_implementation, python_pure_op_implementation

    @python_pure_op_implementation(alpha=lambda node: node.alpha)
    def LeakyRelu(X, Y):
        K.unary(X, Y, L.UN_LEAKYRELU, alpha)  # noqa: F821 - alpha comes from compute

    @op_implementation(op="Softplus", name="composed")
    class ComposedSoftplus(ONNXForward):
        @staticmethod
        def forward(node, state, sdfg):
            ns, nst, ins, outs = empty_sdfg_for_node(sdfg, state, node)
            shape, dtype = ns.arrays["X"].shape, ns.arrays["X"].dtype
            ns.add_transient("e", shape, dtype)
            ns.add_transient("s", shape, dtype)
            ns.add_constant("one", torch.ones((), dtype=dtype))
            ex, add, log = donnx.ONNXExp("exp"), donnx.ONNXAdd("add"), donnx.ONNXLog("log")
            nst.add_edge(ins["X"], None, ex, "input", ns.make_array_memlet("X"))
            nst.add_edge(ex, "output", nst.add_access("e"), None, ns.make_array_memlet("e"))
            nst.add_edge(nst.add_access("e"), None, add, "A", ns.make_array_memlet("e"))
            nst.add_edge(nst.add_read("one"), None, add, "B", ns.make_array_memlet("one"))
            nst.add_edge(add, "C", nst.add_access("s"), None, ns.make_array_memlet("s"))
            nst.add_edge(nst.add_access("s"), None, log, "input", ns.make_array_memlet("s"))
            nst.add_edge(log, "output", outs["Y"], None, ns.make_array_memlet("Y"))
            return ns

    try:
        x = rng.standard_normal((37, 50)).astype(np.float32)
        for op_cls, impl, attrs, want in ((donnx.ONNXLeakyRelu, "pure", dict(alpha=0.2), np.where(x > 0, x, np.float32(0.2) * x)),
                                          (donnx.ONNXSoftplus, "composed", {}, ops.softplus(x))):
            g = sd.SDFG("helper_" + impl)
            g.add_array("x", x.shape, torch.float32)
            g.add_array("y", x.shape, torch.float32)
            st = g.add_state()
            node = op_cls("n0", **attrs)
            node.implementation = impl
            st.add_edge(st.add_read("x"), None, node, "X", g.make_array_memlet("x"))
            st.add_edge(node, "Y", st.add_write("y"), None, g.make_array_memlet("y"))
            comp = g.compile()
            y = empty(x.shape, torch.float32)
            comp(x=dev(x), y=y)
            assert_close(y, want, what=impl)
            assert len(comp.kernel_names()) == (1 if impl == "pure" else 3)
        status_ok()
    finally:
        donnx.ONNXLeakyRelu.implementations.pop("pure", None)
        donnx.ONNXSoftplus.implementations.pop("composed", None)
        ONNXForward.unregister(LeakyRelu)
        ONNXForward.unregister(ComposedSoftplus)


def test_conv_prepacked_weights(rng):
    """``b200ml_conv_prepack``: weights split once give bit-identical results in one launch instead of two, for the 1x1
    and the implicit-GEMM kernel; convolutions on the other kernels report that there is nothing to pack."""
    if os.environ.get("B200ML_CONV_TC", "1") == "0":
        pytest.skip("the tensor-core convolution is switched off")
    for (n, cin, cout, hw, k, pads, strides) in ((8, 24, 144, (56, 56), (1, 1), (0, 0, 0, 0), (1, 1)), (8, 32, 48, (28, 28), (3, 3), (1, 1, 1, 1), (1, 1)),
                                                 (8, 32, 64, (56, 56), (3, 3), (1, 1, 1, 1), (2, 2))):
        x = dev(rng.standard_normal((n, cin) + hw).astype(np.float32))
        w = dev((rng.standard_normal((cout, cin) + k) * 0.1).astype(np.float32))
        b = dev(rng.standard_normal(cout).astype(np.float32))
        oh = (hw[0] + pads[0] + pads[2] - k[0]) // strides[0] + 1
        ow = (hw[1] + pads[1] + pads[3] - k[1]) // strides[1] + 1
        y0, y1 = empty((n, cout, oh, ow), torch.float32), empty((n, cout, oh, ow), torch.float32)
        K.conv2d(x, w, y0, bias=b, strides=strides, pads=pads, act=L.EPI_RELU)
        packed = K.conv_prepack(tuple(x.shape), w, bias=b, strides=strides, pads=pads)
        assert packed is not None and packed.numel() > 0
        before = L.launch_count()
        K.conv2d(x, w, y1, bias=b, strides=strides, pads=pads, act=L.EPI_RELU, packed_weight=packed)
        assert L.launch_count() - before == 1
        assert torch.equal(y0, y1)
    wd = dev(rng.standard_normal((16, 1, 3, 3)).astype(np.float32))
    assert K.conv_prepack((4, 16, 32, 32), wd, pads=(1, 1, 1, 1), group=16) is None            # depthwise
    ws = dev(rng.standard_normal((16, 3, 3, 3)).astype(np.float32))
    assert K.conv_prepack((32, 3, 64, 64), ws, strides=(2, 2)) is None                         # 27 terms: the direct kernel
    status_ok()
