"""Writes ``ref_pure_expansions.npz`` + ``ref_pure_expansions.json``: outputs of the reference's OWN pure expansions.

    python tests/golden/generate_from_reference.py <path to a DaCeML checkout>

Every vector here comes from the reference's source files
(``daceml/onnx/op_implementations/pure_implementations.py`` and ``img_op_implementations.py``), imported unchanged
and executed under numpy by ``reference_harness.py`` (no DaCe, no onnx): the bodies of the
``@python_pure_op_implementation`` functions, the Einsum equations and mapped tasklets that ``PureMatMul`` /
``PureGemm`` / ``PureSum`` / ``PureCast`` / ``PureGather`` build, the subset copies of ``SplitPure`` /
``PureSliceAllConstant``, and the loop nest of ``PureConv2D``.  Shapes follow the reference's tests
(``tests/pure_expansions/test_expansions.py``, ``test_conv_expansion.py``; convolutions on 2 images of 16 x 16
instead of 8 of 32 x 32, because the loop nest runs as Python), plus the operator forms the five benchmark
configurations use.  ``tests/test_oracle.py`` checks the CPU oracle against these vectors and the GPU tests check
the kernels against them.

The JSON manifest lists, per case: the operator, the implementation name, the node's attributes, the connector
names of inputs and outputs (array ``<case>:<connector>`` in the ``.npz``) and which inputs are model constants.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import reference_harness as H  # noqa: E402

CASES, ARRAYS = [], {}


def case(name, op, inputs, outputs, implementation="pure", constants=(), **attrs):
    result = H.run(op, inputs, outputs, implementation=implementation, constants=constants, **attrs)
    for k, v in inputs.items():
        ARRAYS["%s:%s" % (name, k)] = np.asarray(v)
    for k, v in result.items():
        ARRAYS["%s:%s" % (name, k)] = v
    CASES.append({"case": name, "op": op, "implementation": implementation, "attrs": attrs, "inputs": list(inputs),
                  "outputs": list(result), "constants": list(constants)})
    return result


def f32(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


def main(reference_root):
    H.install(reference_root)
    rng = np.random.default_rng(20241125)
    F = np.float32
    x = f32(rng, 2, 4, 10)

    # ---- unary, test_expansions.py:354 uses normal(scale=10) on [2, 4, 10] ----
    for op, inp, out, data, attrs in [
            ("Log", "input", "output", np.abs(x) + F(0.1), {}), ("Exp", "input", "output", x, {}),
            ("Sqrt", "X", "Y", np.abs(x), {}), ("Tanh", "input", "output", x, {}), ("Erf", "input", "output", x, {}),
            ("Relu", "X", "Y", x, {}), ("LeakyRelu", "X", "Y", x, {"alpha": 0.01}), ("Sigmoid", "X", "Y", x * F(3), {}),
            ("Softplus", "X", "Y", x * F(3), {}), ("Reciprocal", "X", "Y", f32(rng, 2, 4, 10, scale=10), {}),
            ("Identity", "input", "output", x, {})]:
        case(op.lower(), op, {inp: data}, {out: (data.shape, F)}, **attrs)
    case("clip", "Clip", {"input": x, "min": np.array(-0.5, F), "max": np.array(0.75, F)}, {"output": (x.shape, F)},
         constants=("min", "max"))
    case("expand_noop", "Expand", {"input": x, "shape": np.array(x.shape, np.int64)}, {"output": (x.shape, F)})

    # ---- binary with numpy broadcasting ----
    y_same, y_row, y_scalar = f32(rng, 2, 4, 10), f32(rng, 10), np.array(2.0, F)
    for op in ("Add", "Sub", "Mul", "Div"):
        for tag, other in (("same", y_same), ("row", y_row), ("scalar", np.array(0.125, F))):
            other = np.abs(other) + F(0.5) if op == "Div" else other
            case("%s_%s" % (op.lower(), tag), op, {"A": x, "B": other}, {"C": (x.shape, F)})
    case("pow_scalar", "Pow", {"X": x, "Y": y_scalar}, {"Z": (x.shape, F)})
    case("pow_same", "Pow", {"X": np.abs(x) + F(0.1), "Y": y_same}, {"Z": (x.shape, F)})
    cond = rng.random((2, 4, 10)) > 0.5
    case("where", "Where", {"condition": cond, "X": x, "Y": y_same}, {"output": (x.shape, F)})
    case("sum3", "Sum", {"data_0__0": x, "data_0__1": y_same, "data_0__2": f32(rng, 2, 4, 10)}, {"sum": (x.shape, F)})

    # ---- reductions, test_expansions.py:187-237 (normal(scale=10), [2, 4, 10]) and :240-278 (full reduction) ----
    xr = f32(rng, 2, 4, 10, scale=10)
    for kind, keep, axes in [("Sum", True, [0]), ("Sum", False, [-1]), ("Sum", True, [0, -1]), ("Max", False, [0, -1]),
                             ("Max", True, [0]), ("Max", True, [-1]), ("Mean", True, [-1]), ("Mean", True, [0, -1]),
                             ("Mean", False, [0]), ("Min", True, [1]), ("Min", False, [0, -1])]:
        shape = getattr(np, kind.lower())(xr, axis=tuple(axes), keepdims=keep).shape
        case("reduce%s_%d_%s" % (kind.lower(), keep, "_".join(str(a) for a in axes).replace("-", "m")), "Reduce" + kind,
             {"data": xr}, {"reduced": (shape, F)}, axes=axes, keepdims=int(keep))
    case("reducemean_scalar", "ReduceMean", {"data": xr}, {"reduced": ((1,), F)}, axes=None, keepdims=0)
    case("global_average_pool", "GlobalAveragePool", {"X": f32(rng, 2, 5, 7, 7)}, {"Y": ((2, 5, 1, 1), F)})

    # ---- Softmax / LogSoftmax: reduction over the axes [axis:] ----
    for op in ("Softmax", "LogSoftmax"):
        for axis in (0, 1, 2, -1):
            case("%s_axis%s" % (op.lower(), str(axis).replace("-", "m")), op, {"input": x * F(2)}, {"output": (x.shape, F)}, axis=axis)
        scores = f32(rng, 2, 4, 8, 8, scale=3)
        case("%s_scores" % op.lower(), op, {"input": scores}, {"output": (scores.shape, F)}, axis=3)
        logits = f32(rng, 16, 10, scale=2)
        case("%s_logits" % op.lower(), op, {"input": logits}, {"output": (logits.shape, F)}, axis=1)

    # ---- data movement ----
    t = f32(rng, 2, 3, 4, 5)
    case("transpose_default", "Transpose", {"data": t}, {"transposed": ((5, 4, 3, 2), F)}, perm=None)
    case("transpose_heads", "Transpose", {"data": t}, {"transposed": ((2, 4, 3, 5), F)}, perm=[0, 2, 1, 3])
    case("transpose_keys", "Transpose", {"data": t}, {"transposed": ((2, 4, 5, 3), F)}, perm=[0, 2, 3, 1])
    case("transpose_einsum", "Transpose", {"data": t}, {"transposed": ((2, 4, 3, 5), F)}, implementation="einsum", perm=[0, 2, 1, 3])
    for shape in ([8, 10], [80], [2, 40]):  # test_expansions.py:282-318
        case("reshape_%s" % "x".join(map(str, shape)), "Reshape", {"data": xr, "shape": np.array(shape, np.int64)},
             {"reshaped": (tuple(shape), F)})
    case("flatten", "Flatten", {"input": xr}, {"output": ((2, 40), F)}, axis=1)  # :320-351
    case("unsqueeze", "Unsqueeze", {"data": f32(rng, 3, 3)}, {"expanded": ((3, 1, 3, 1), F)}, axes=[1, 3])  # :565-585
    case("shape", "Shape", {"data": rng.random((9, 5, 3))}, {"shape": ((3,), np.int64)})  # :463-478
    xi = rng.integers(0, 10, size=(2, 4)).astype(np.int32)  # casts: :85-184
    xf = f32(rng, 2, 4, scale=10)
    case("cast_int_to_float", "Cast", {"input": xi}, {"output": ((2, 4), F)}, to=np.float32)
    case("cast_float_to_int", "Cast", {"input": xf}, {"output": ((2, 4), np.int32)}, to=np.int32)
    case("cast_float_to_long", "Cast", {"input": xf}, {"output": ((2, 4), np.int64)}, to=np.int64)
    case("cast_same", "Cast", {"input": xf}, {"output": ((2, 4), F)}, to=np.float32)
    # Gather: :480-562
    case("gather_onnx_1", "Gather", {"data": np.array([[1.0, 1.2], [2.3, 3.4], [4.5, 5.7]]), "indices": np.array([[0, 1], [1, 2]])},
         {"output": ((2, 2, 2), np.float64)}, axis=0)
    embs, ids = rng.random((64, 8)), rng.integers(0, 64, size=(8, 16))
    case("gather_bert", "Gather", {"data": embs, "indices": ids}, {"output": ((8, 16, 8), np.float64)}, axis=0)
    case("gather_scalar", "Gather", {"data": rng.random((1, 8, 32)), "indices": np.array(0, np.int64)},
         {"output": ((1, 32), np.float64)}, axis=1)
    case("gather_onnx_2", "Gather", {"data": np.array([[1.0, 1.2, 1.9], [2.3, 3.4, 3.9], [4.5, 5.7, 5.9]]), "indices": np.array([[0, 2]])},
         {"output": ((3, 1, 2), np.float64)}, axis=1)
    sp = f32(rng, 6, 8)
    case("split_axis1", "Split", {"input": sp}, {"outputs__0": ((6, 3), F), "outputs__1": ((6, 5), F)}, axis=1, split=[3, 5])
    case("split_axis0", "Split", {"input": sp}, {"outputs__0": ((2, 8), F), "outputs__1": ((4, 8), F)}, axis=0, split=[2, 4])
    i64 = lambda *v: np.array(v, np.int64)
    case("slice_axis1", "Slice", {"data": sp, "starts": i64(2), "ends": i64(7), "axes": i64(1), "steps": i64(1)},
         {"output": ((6, 5), F)}, constants=("starts", "ends", "axes", "steps"))
    case("slice_two_axes_step", "Slice", {"data": sp, "starts": i64(1, 0), "ends": i64(5, 2 ** 62), "axes": i64(0, 1), "steps": i64(1, 2)},
         {"output": ((4, 4), F)}, constants=("starts", "ends", "axes", "steps"))

    # ---- MatMul / Gemm / Einsum ----
    for tag, a_shape, b_shape in [("2d", (2, 4), (4, 3)), ("3d_2d", (3, 5, 8), (8, 6)), ("4d_4d", (2, 3, 16, 8), (2, 3, 8, 24)),
                                  ("2d_3d", (5, 40), (3, 40, 24))]:
        a, b = rng.random(a_shape).astype(F), rng.random(b_shape).astype(F)
        case("matmul_" + tag, "MatMul", {"A": a, "B": b}, {"Y": (np.matmul(a, b).shape, F)})
    ga, gb = f32(rng, 8, 16), f32(rng, 16, 12)
    for tag, ta, tb, alpha, beta, c_shape in [("plain", 0, 0, 1.0, 1.0, (12,)), ("linear", 0, 1, 1.0, 1.0, (12,)),
                                              ("scaled", 1, 0, 0.5, 2.0, (8, 12)), ("both_t", 1, 1, 1.5, 0.5, (12,)),
                                              ("no_c", 0, 1, 1.0, 0.0, None)]:  # alpha != 1 with beta == 0 is not
        # expressible: the expansion only declares its "scaled" array when beta != 0 (pure_implementations.py:493-496)
        a = ga.T.copy() if ta else ga
        b = gb.T.copy() if tb else gb
        ins = {"A": a, "B": b}
        if c_shape is not None:
            ins["C"] = f32(rng, *c_shape)
        case("gemm_" + tag, "Gemm", ins, {"Y": ((8, 12), F)}, transA=ta, transB=tb, alpha=alpha, beta=beta)
    ea, eb = rng.random((5, 4, 3)), rng.random((3, 2))  # test_expansions.py:387-405, float64
    case("einsum_bij_jk", "Einsum", {"Inputs__0": ea, "Inputs__1": eb}, {"Output": ((5, 4, 2), np.float64)}, equation="bij, jk -> bik")
    q, k = f32(rng, 2, 4, 8, 16), f32(rng, 2, 4, 8, 16)
    case("einsum_qk", "Einsum", {"Inputs__0": q, "Inputs__1": k}, {"Output": ((2, 4, 8, 8), F)}, equation="bhid,bhjd->bhij")
    p = f32(rng, 2, 4, 8, 8)
    case("einsum_pv", "Einsum", {"Inputs__0": p, "Inputs__1": k}, {"Output": ((2, 4, 8, 16), F)}, equation="bhij,bhjd->bhid")

    # ---- Conv: test_conv_expansion.py:9-66 (uniform [0,1) data), and the 1x1 form of the MBConv block ----
    for cin, ksize, filters, bias in [(1, (3, 3), 8, True), (8, (3, 3), 3, False), (8, (5, 5), 3, True), (8, (4, 4), 3, False)]:
        X, W = rng.random((2, cin, 16, 16)).astype(F), rng.random((filters, cin) + ksize).astype(F)
        ins = {"X": X, "W": W}
        if bias:
            ins["B"] = rng.random(filters).astype(F)
        case("conv_c%d_k%d_f%d" % (cin, ksize[0], filters), "Conv", ins, {"Y": ((2, filters, 17 - ksize[0], 17 - ksize[1]), F)},
             group=1, dilations=None, pads=None, strides=None, auto_pad="NOTSET", kernel_shape=None)
    X, W = f32(rng, 2, 24, 6, 6), f32(rng, 40, 24, 1, 1, scale=0.05)
    case("conv_pointwise", "Conv", {"X": X, "W": W, "B": f32(rng, 40, scale=0.05)}, {"Y": ((2, 40, 6, 6), F)},
         group=1, dilations=[1, 1], pads=[0, 0, 0, 0], strides=[1, 1], auto_pad="NOTSET", kernel_shape=[1, 1])

    # ---- the decomposed LayerNorm and GELU sub-graphs of the exported BERT layer, node by node ----
    h = f32(rng, 2, 6, 32)
    gamma, beta = (1 + f32(rng, 32, scale=0.1)), f32(rng, 32, scale=0.1)
    S = h.shape
    mean = case("ln_1_mean", "ReduceMean", {"data": h}, {"reduced": ((2, 6, 1), F)}, axes=[-1], keepdims=1)["reduced"]
    cen = case("ln_2_sub", "Sub", {"A": h, "B": mean}, {"C": (S, F)})["C"]
    sq = case("ln_3_pow", "Pow", {"X": cen, "Y": np.array(2.0, F)}, {"Z": (S, F)})["Z"]
    var = case("ln_4_mean", "ReduceMean", {"data": sq}, {"reduced": ((2, 6, 1), F)}, axes=[-1], keepdims=1)["reduced"]
    ve = case("ln_5_add", "Add", {"A": var, "B": np.array(1e-12, F)}, {"C": ((2, 6, 1), F)})["C"]
    sd = case("ln_6_sqrt", "Sqrt", {"X": ve}, {"Y": ((2, 6, 1), F)})["Y"]
    nrm = case("ln_7_div", "Div", {"A": cen, "B": sd}, {"C": (S, F)})["C"]
    scl = case("ln_8_mul", "Mul", {"A": nrm, "B": gamma}, {"C": (S, F)})["C"]
    out = case("ln_9_add", "Add", {"A": scl, "B": beta}, {"C": (S, F)})["C"]
    ARRAYS["layernorm_chain:x"], ARRAYS["layernorm_chain:gamma"], ARRAYS["layernorm_chain:beta"] = h, gamma, beta
    ARRAYS["layernorm_chain:y"] = out
    g0 = f32(rng, 2, 6, 32, scale=2)
    d = case("gelu_1_div", "Div", {"A": g0, "B": np.array(1.4142135381698608, F)}, {"C": (S, F)})["C"]
    e = case("gelu_2_erf", "Erf", {"input": d}, {"output": (S, F)})["output"]
    a1 = case("gelu_3_add", "Add", {"A": e, "B": np.array(1.0, F)}, {"C": (S, F)})["C"]
    m1 = case("gelu_4_mul", "Mul", {"A": g0, "B": a1}, {"C": (S, F)})["C"]
    m2 = case("gelu_5_mul", "Mul", {"A": m1, "B": np.array(0.5, F)}, {"C": (S, F)})["C"]
    ARRAYS["gelu_chain:x"], ARRAYS["gelu_chain:y"] = g0, m2

    # ---- Conv large enough for the implicit-GEMM tensor-core kernel (64 terms or more, 4096 output pixels): the
    # reference's stride-1, unpadded loop nest on 4 images; 5x5 on a width the TMA unit can describe, 3x3 on one it
    # cannot.  These two take about a minute each (the loop nest runs as Python).  Drawn from a generator of their own so
    # that the cases above keep their values.
    rng2 = np.random.default_rng(20261)
    for cin, ksize, filters, hw in [(4, (5, 5), 16, (36, 36)), (8, (3, 3), 16, (34, 34))]:
        X = rng2.random((4, cin) + hw).astype(F)
        W = (rng2.random((filters, cin) + ksize).astype(F) - np.float32(0.5))
        B = rng2.random(filters).astype(F)
        case("conv_igemm_c%d_k%d_f%d" % (cin, ksize[0], filters), "Conv", {"X": X, "W": W, "B": B},
             {"Y": ((4, filters, hw[0] + 1 - ksize[0], hw[1] + 1 - ksize[1]), F)},
             group=1, dilations=None, pads=None, strides=None, auto_pad="NOTSET", kernel_shape=None)

    # ---- and a 1x1 convolution large enough for the 1x1 tensor-core kernel (16384 pixels) ----
    X = rng2.standard_normal((4, 8, 64, 64)).astype(F)
    W = (rng2.standard_normal((8, 8, 1, 1)) * 0.3).astype(F)
    case("conv_pointwise_tc", "Conv", {"X": X, "W": W, "B": rng2.standard_normal(8).astype(F)}, {"Y": ((4, 8, 64, 64), F)},
         group=1, dilations=[1, 1], pads=[0, 0, 0, 0], strides=[1, 1], auto_pad="NOTSET", kernel_shape=[1, 1])

    def plain(v):
        if isinstance(v, type):
            return np.dtype(v).name
        return v

    for c in CASES:
        c["attrs"] = {k: plain(v) for k, v in c["attrs"].items()}
    np.savez_compressed(os.path.join(HERE, "ref_pure_expansions.npz"), **ARRAYS)
    with open(os.path.join(HERE, "ref_pure_expansions.json"), "w") as f:
        json.dump({"source": "daceml/onnx/op_implementations/{pure,img_op}_implementations.py executed under numpy",
                   "chains": ["layernorm_chain", "gelu_chain"], "cases": CASES}, f, indent=1)
    print("wrote %d cases, %d arrays" % (len(CASES), len(ARRAYS)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
