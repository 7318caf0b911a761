"""Pins the CPU oracle: against the committed golden vectors, against numpy / PyTorch on the shapes
the reference's own tests use, and the timed C restatement against the numpy one."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import cpu_baseline, ops

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def test_matmul_reference_shape():
    # tests/pure_expansions/test_expansions.py:23-63
    g = gold("matmul")
    np.testing.assert_allclose(ops.matmul(g["a"], g["b"]), g["y"], rtol=1e-6)
    np.testing.assert_allclose(g["y"], g["a"] @ g["b"], rtol=1e-5, atol=1e-8)
    np.testing.assert_allclose(ops.matmul(g["a4"], g["b4"]), g["y4"], rtol=1e-6, atol=1e-6)


def test_matmul_equation_strings():
    # letters are popped from the end of [z, y, ..., a] (pure_implementations.py:133-136, 172-186)
    assert ops.matmul_equation((8, 512, 1024), (1024, 1024)) == "aik,kj->aij"
    assert ops.matmul_equation((8, 16, 512, 64), (8, 16, 64, 512)) == "baik,bakj->baij"
    assert ops.matmul_equation((4, 8), (8, 3), trans_b=True) == "ik,jk->ij"
    with pytest.raises(ValueError):
        ops.matmul(np.zeros(5, np.float32), np.zeros((5, 6), np.float32))  # 1-D operands are rejected


def test_einsum_reference_case():
    # tests/pure_expansions/test_expansions.py:387-405
    g = gold("einsum")
    np.testing.assert_allclose(ops.einsum("bij, jk -> bik", g["a"], g["b"]), g["y"], rtol=1e-6)
    with pytest.raises(ValueError):
        ops.einsum("...ij,jk->...ik", g["a"], g["b"])


def test_gemm_rules():
    g = gold("gemm")
    np.testing.assert_allclose(ops.gemm(g["a"], g["b"], g["c"], alpha=0.5, beta=2.0, trans_b=1), g["y"], rtol=1e-6)
    np.testing.assert_allclose(ops.gemm(g["at"], g["bt"], g["c2"], trans_a=1), g["y2"], rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError):  # C[1, N] is not broadcast (pure_implementations.py:533-539)
        ops.gemm(g["a"], g["b"], g["c"][None, :], trans_b=1)


@pytest.mark.parametrize("kind, keep, axes", [("sum", True, [0]), ("sum", False, [-1]), ("sum", True, [0, -1]),
                                              ("max", False, [0, -1]), ("max", True, [0]), ("max", True, [-1]),
                                              ("mean", True, [-1]), ("mean", True, [0, -1]), ("mean", False, [0])])
def test_reduce_reference_cases(kind, keep, axes):
    # tests/pure_expansions/test_expansions.py:187-237
    g = gold("reduce")
    out = getattr(ops, "reduce_" + kind)(g["x"], axes, keep)
    key = "%s_%d_%s" % (kind, int(keep), "_".join(str(a) for a in axes))
    np.testing.assert_allclose(out, g[key], rtol=1e-6)
    np.testing.assert_allclose(out, getattr(np, kind)(g["x"], axis=tuple(axes), keepdims=keep), rtol=1e-5, atol=1e-5)


def test_softmax_axis_semantics():
    g = gold("softmax")
    np.testing.assert_allclose(ops.softmax(g["x"], 3), g["softmax_axis3"], rtol=1e-6)
    np.testing.assert_allclose(ops.softmax(g["x"], 1), g["softmax_axis1"], rtol=1e-6)
    assert abs(float(ops.softmax(g["x"], 1)[0].sum()) - 1.0) < 1e-5  # joint over all axes from 1 on
    np.testing.assert_allclose(ops.softmax(g["x"], -1), g["softmax_axis3"], rtol=1e-6)
    np.testing.assert_allclose(ops.log_softmax(g["x"][0, 0], 1), g["logsoftmax"], rtol=1e-6, atol=1e-6)


def test_elementwise_golden():
    g = gold("elementwise")
    x, y = g["x"], g["y"]
    for name, val in [("add", ops.add(x, y)), ("sub", ops.sub(x, y)), ("mul", ops.mul(x, y)), ("div", ops.div(x, y)),
                      ("erf", ops.erf(x)), ("tanh", ops.tanh(x)), ("relu", ops.relu(x)), ("sigmoid", ops.sigmoid(x)),
                      ("gelu", ops.gelu_chain(x)), ("swish", ops.swish(x)), ("leaky", ops.leaky_relu(x, 0.1))]:
        np.testing.assert_allclose(val, g[name], rtol=1e-6, atol=1e-7, err_msg=name)


@pytest.mark.parametrize("idx, bias", [(0, True), (1, False), (2, True), (3, False)])
def test_conv_reference_cases(idx, bias):
    # tests/pure_expansions/test_conv_expansion.py:9-66 compares with F.conv2d under np.allclose defaults
    g = gold("conv")
    x, w = g["x%d" % idx], g["w%d" % idx]
    b = g["b%d" % idx] if bias else None
    y = ops.conv2d(x, w, b)
    np.testing.assert_allclose(y, g["y%d" % idx], rtol=1e-6, atol=1e-6)
    ref = F.conv2d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b) if bias else None).numpy()
    assert np.allclose(ref, y)
    assert ops.conv_pure_supported(x.shape, w.shape, (1, 1), (0, 0, 0, 0), (1, 1), 1)
    np.testing.assert_allclose(cpu_baseline.conv2d(x, w, b), y, rtol=1e-5, atol=1e-5)


def test_conv_generalised_forms():
    g = gold("conv")
    np.testing.assert_allclose(ops.conv2d(g["xs"], g["ws"], strides=(2, 2)), g["ys"], rtol=1e-6, atol=1e-6)
    assert not ops.conv_pure_supported(g["xs"].shape, g["ws"].shape, (2, 2), (0, 0, 0, 0), (1, 1), 1)
    np.testing.assert_allclose(cpu_baseline.conv2d(g["xs"], g["ws"], strides=(2, 2)), g["ys"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(cpu_baseline.conv2d(g["xd"], g["wd"], pads=(1, 1, 1, 1), group=12), g["yd"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(ops.global_average_pool(g["xd"]), g["gap"], rtol=1e-6)


def test_graph_oracles_against_golden():
    g = gold("mlp")
    np.testing.assert_allclose(ops.mlp(g["x"], {k: g[k] for k in ("w1", "b1", "w2", "b2", "w3", "b3")}), g["y"], rtol=1e-5, atol=1e-6)
    g = gold("mbconv")
    p = {k: g[k] for k in g.files if k not in ("x", "y")}
    np.testing.assert_allclose(ops.mbconv_block(g["x"], p), g["y"], rtol=1e-5, atol=1e-6)
    g = gold("bert_layer")
    p = {k: g[k] for k in g.files if k not in ("x", "y_fp32", "y_fp16")}
    np.testing.assert_allclose(ops.bert_layer(g["x"], p, heads=2, store=np.float32), g["y_fp32"], rtol=1e-5, atol=1e-5)
    y16 = ops.bert_layer(g["x"], p, heads=2, store=np.float16).astype(np.float32)
    np.testing.assert_allclose(y16, g["y_fp16"], rtol=1e-3, atol=1e-3)
    # the fp16 storage rule stays within the fp16 tolerance of the fp32 result
    np.testing.assert_allclose(y16, g["y_fp32"], rtol=2e-2, atol=2e-2)


def test_c_restatement_matches_numpy_oracle():
    g = gold("bert_layer")
    p = {k: torch.from_numpy(g[k]) for k in g.files if k not in ("x", "y_fp32", "y_fp16")}
    y = cpu_baseline.CpuBertLayer(p, heads=2).forward(torch.from_numpy(g["x"]))
    np.testing.assert_allclose(y.numpy(), g["y_fp32"], rtol=1e-4, atol=1e-5)


def test_data_movement_reference_cases():
    # tests/pure_expansions/test_expansions.py:464-563: Shape, the two Gather examples of the ONNX operator docs, the
    # embedding lookup and the scalar-index Gather of a BERT model -- each compared with numpy indexing, as there
    rng = np.random.default_rng(3)
    assert ops.shape(np.zeros((9, 5, 3))).tolist() == [9, 5, 3]
    d = np.array([[1.0, 1.2], [2.3, 3.4], [4.5, 5.7]])
    idx = np.array([[0, 1], [1, 2]])
    assert np.array_equal(ops.gather(d, idx, 0), d[idx])
    assert ops.gather(d, idx, 0).tolist() == [[[1.0, 1.2], [2.3, 3.4]], [[2.3, 3.4], [4.5, 5.7]]]
    embs, ids = rng.random((64, 8)), rng.integers(0, 64, (8, 16))
    assert np.array_equal(ops.gather(embs, ids, 0), embs[ids])
    d3 = rng.random((1, 8, 32))
    assert np.array_equal(ops.gather(d3, np.int64(5), 1), np.take(d3, 5, axis=1))
    d2 = np.array([[1.0, 1.2, 1.9], [2.3, 3.4, 3.9], [4.5, 5.7, 5.9]])
    assert ops.gather(d2, np.array([[0, 2]]), 1).tolist() == [[[1.0, 1.9]], [[2.3, 3.9]], [[4.5, 5.9]]]
    # Slice as the reference expands it (axis 0, step 1, INT64_MAX end) and the general form against numpy
    x = rng.standard_normal((6, 7, 8)).astype(np.float32)
    assert np.array_equal(ops.slice_(x, [2], [(1 << 63) - 1], [0], [1]), x[2:])
    assert np.array_equal(ops.slice_(x, [1, -5], [4, 100], [1, 2], [2, 3]), x[:, 1:4:2, -5::3])
    parts = ops.split(x, 1, [3, 4])
    assert [p.shape for p in parts] == [(6, 3, 8), (6, 4, 8)] and np.array_equal(ops.concat(parts, 1), x)
    assert np.array_equal(ops.expand(x[:, :1], (2, 6, 7, 8)), np.broadcast_to(x[:, :1], (2, 6, 7, 8)))
    c = rng.integers(0, 2, (6, 1, 8)).astype(bool)
    assert np.array_equal(ops.where(c, x, np.float32(0)), np.where(c, x, 0).astype(np.float32))
    # MaxPool against PyTorch (no padding is the reference's case; padded windows agree too)
    img = rng.standard_normal((2, 3, 9, 8)).astype(np.float32)
    assert np.array_equal(ops.maxpool2d(img, (2, 2), (2, 2)), F.max_pool2d(torch.from_numpy(img), 2, 2).numpy())
    assert np.array_equal(ops.maxpool2d(img, (3, 2), (2, 1), (1, 1, 1, 1)),
                          F.max_pool2d(torch.from_numpy(img), (3, 2), (2, 1), padding=(1, 1)).numpy())


# ------------------------------------------------------------------------------------------------
# The oracle against outputs of the reference's own source: tests/golden/ref_pure_expansions.* hold
# what pure_implementations.py / img_op_implementations.py compute when their bodies are executed
# under numpy (tests/golden/generate_from_reference.py).
# ------------------------------------------------------------------------------------------------
import ref_cases  # noqa: E402
from ref_cases import REF_CASES, ref_arrays, oracle_outputs  # noqa: E402


@pytest.mark.parametrize("case", REF_CASES, ids=[c["case"] for c in REF_CASES])
def test_oracle_matches_reference_source(case):
    arrays = ref_arrays()
    got = oracle_outputs(case, arrays)
    assert set(got) == set(case["outputs"])
    for conn, value in got.items():
        want = arrays["%s:%s" % (case["case"], conn)]
        assert value.shape == want.shape and value.dtype == want.dtype, (conn, value.shape, want.shape, value.dtype, want.dtype)
        if not np.issubdtype(want.dtype, np.floating) or case["op"] in ref_cases.BIT_EXACT_OPS:
            assert np.array_equal(value, want), conn
        else:
            # the same arithmetic in the same type; only the order of a reduction's additions (numpy pairwise against
            # np.einsum / sequential) and libm-vs-numpy rounding of exp / erf / tanh may differ: a few ulp
            np.testing.assert_allclose(value, want, rtol=2e-6, atol=1e-6 * max(1.0, float(np.abs(want).max())))


def test_reference_chains_match_oracle_graphs():
    """The decomposed LayerNorm and GELU sub-graphs, evaluated node by node with the reference's bodies."""
    a = ref_arrays()
    ln = ops.layernorm_chain(a["layernorm_chain:x"], a["layernorm_chain:gamma"], a["layernorm_chain:beta"], eps=1e-12)
    np.testing.assert_allclose(ln, a["layernorm_chain:y"], rtol=2e-6, atol=2e-6)
    np.testing.assert_allclose(ops.gelu_chain(a["gelu_chain:x"]), a["gelu_chain:y"], rtol=2e-6, atol=1e-6)
