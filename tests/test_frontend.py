"""Host logic of the drop-in boundary: registry, selection levels, validation, expansion planning."""
import numpy as np
import pytest
import torch

import daceml_b200.onnx as donnx
from daceml_b200 import graphs, sdfg as sd
from daceml_b200.onnx import ONNXForward, op_implementation
from daceml_b200.onnx.op_implementations import b200_implementations as impl
from daceml_b200.sdfg import KernelTasklet
from daceml_b200.util import utils


def one_node_sdfg(node, ins, outs):
    g = sd.SDFG("t")
    st = g.add_state()
    st.add_node(node)
    for conn, (name, shape, dt) in ins.items():
        g.add_array(name, shape, dt)
        st.add_edge(st.add_access(name), None, node, conn, g.make_array_memlet(name))
    for conn, (name, shape, dt) in outs.items():
        g.add_array(name, shape, dt)
        st.add_edge(node, conn, st.add_access(name), None, g.make_array_memlet(name))
    return g, st


def test_registry_lists_b200_implementations():
    for op in ("MatMul", "Gemm", "Einsum", "Conv", "Softmax", "LogSoftmax", "Add", "Mul", "Erf", "ReduceMean", "Transpose",
               "GlobalAveragePool", "Sigmoid", "Relu"):
        names = [n for n, _ in ONNXForward.registered_implementations(op)]
        assert "b200" in names, op
        assert donnx.has_onnx_node(op)
        assert "b200" in donnx.get_onnx_node(op).implementations
    assert donnx.default_implementation == "b200"


def test_late_registration_reaches_the_node_class():
    calls = []

    @op_implementation(op="Tanh", name="probe")
    class ProbeTanh(ONNXForward):
        @staticmethod
        def forward_can_be_applied(node, state, sdfg):
            return True

        @staticmethod
        def forward(node, state, sdfg):
            calls.append(node.label)
            return KernelTasklet(node.label, lambda i, o: None)

    try:
        assert ("probe", ProbeTanh) in ONNXForward.registered_implementations("Tanh")
        assert "Implementation name" in ProbeTanh.__doc__
        node = donnx.ONNXTanh("t")
        g, st = one_node_sdfg(node, {"input": ("x", (4, ), np.float32)}, {"output": ("y", (4, ), np.float32)})
        node.implementation = "probe"  # per-instance selection
        assert node.expand(g, st) == "probe"
        assert calls == ["t"]
        # per-class selection
        node2 = donnx.ONNXTanh("t2")
        g2, st2 = one_node_sdfg(node2, {"input": ("x", (4, ), np.float32)}, {"output": ("y", (4, ), np.float32)})
        donnx.ONNXTanh.default_implementation = "probe"
        assert node2.expand(g2, st2) == "probe"
    finally:
        donnx.ONNXTanh.default_implementation = None
        ONNXForward.unregister(ProbeTanh)
        donnx.ONNXTanh.implementations.pop("probe", None)


def test_no_fallback_when_implementation_cannot_be_applied():
    node = donnx.ONNXMatMul("mm")
    g, st = one_node_sdfg(node, {"A": ("a", (5, ), np.float32), "B": ("b", (5, 6), np.float32)}, {"Y": ("y", (6, ), np.float32)})
    with pytest.raises(NotImplementedError):  # 1-D operand: the reference would fall back to ORT here
        node.expand(g, st)
    node = donnx.ONNXAdd("add")
    g, st = one_node_sdfg(node, {"A": ("a", (4, ), np.int64), "B": ("b", (4, ), np.int64)}, {"C": ("c", (4, ), np.int64)})
    with pytest.raises(NotImplementedError):
        node.expand(g, st)


def test_validate_reports_missing_and_unknown_connectors():
    node = donnx.ONNXConv("c")
    g, st = one_node_sdfg(node, {"X": ("x", (1, 1, 4, 4), np.float32)}, {"Y": ("y", (1, 1, 2, 2), np.float32)})
    with pytest.raises(ValueError, match="'W' is not connected"):
        node.expand(g, st)
    node = donnx.ONNXRelu("r")
    g, st = one_node_sdfg(node, {"X": ("x", (4, ), np.float32), "Q": ("q", (4, ), np.float32)}, {"Y": ("y", (4, ), np.float32)})
    with pytest.raises(ValueError, match="unknown input connector"):
        node.expand(g, st)
    with pytest.raises(TypeError):
        donnx.ONNXConv("c", stride=[2, 2])  # attribute names come from the schema


def test_descriptor_helpers_and_attributes():
    node = donnx.ONNXConv("c", strides=[2, 2], group=1)
    g, st = one_node_sdfg(node, {"X": ("x", (32, 3, 64, 64), np.float32), "W": ("w", (16, 3, 3, 3), np.float32)},
                          {"Y": ("y", (32, 16, 31, 31), np.float32)})
    assert utils.in_desc_with_name(node, st, g, "X").shape == (32, 3, 64, 64)
    assert utils.out_desc_with_name(node, st, g, "Y").dtype == torch.float32
    assert node.strides == [2, 2] and node.pads is None and node.auto_pad == "NOTSET"
    g.expand_library_nodes()
    (tasklet, ) = st.topological_compute_nodes()
    assert isinstance(tasklet, KernelTasklet) and tasklet.kernels == ("conv2d", )


def test_gemm_c_broadcast_rule_is_the_references():
    node = donnx.ONNXGemm("g", transB=1)
    g, st = one_node_sdfg(node, {"A": ("a", (4, 8), np.float32), "B": ("b", (3, 8), np.float32), "C": ("c", (1, 3), np.float32)},
                          {"Y": ("y", (4, 3), np.float32)})
    with pytest.raises(ValueError, match="Could not broadcast"):
        node.expand(g, st)


@pytest.mark.parametrize("eq, shapes, expect", [
    ("bij,jk->bik", [(5, 3, 4), (4, 6)], dict(kind="gemm", batch=1, m=15, n=6, k=4, a_layout=0, b_layout=0)),
    ("zik,kj->zij", [(8, 512, 64), (64, 32)], dict(kind="gemm", batch=1, m=4096, n=32, k=64)),
    ("bik,bjk->bij", [(4, 16, 8), (4, 12, 8)], dict(kind="gemm", batch=4, m=16, n=12, k=8, b_layout=1)),
    ("yzik,yzkj->yzij", [(2, 3, 16, 8), (2, 3, 8, 24)], dict(kind="gemm", batch=6, m=16, n=24, k=8)),
    ("ki,kj->ij", [(8, 4), (8, 3)], dict(kind="gemm", a_layout=1, b_layout=0, m=4, n=3, k=8)),
    ("abcd->acbd", [(2, 3, 4, 5)], dict(kind="permute", perm=[0, 2, 1, 3])),
])
def test_einsum_plans(eq, shapes, expect):
    plan = impl._parse_einsum(eq, shapes)
    assert plan is not None
    for k, v in expect.items():
        assert plan[k] == v, (k, plan)


def test_einsum_rejects_what_it_cannot_run():
    assert impl._parse_einsum("...ij,jk->...ik", [(2, 3, 4), (4, 5)]) is None
    assert impl._parse_einsum("ij,jk,kl->il", [(2, 3), (3, 4), (4, 5)]) is None
    assert impl._parse_einsum("ii->i", [(3, 3)]) is None
    assert impl._parse_einsum("ij,kl->ijkl", [(2, 3), (4, 5)]) is None


def test_reduce_axis_grouping():
    assert impl._reduce_groups([2, 4, 10], [0, -1]) == [[2], [0]]
    assert impl._reduce_groups([2, 4, 10], [1, 2]) == [[1, 2]]
    assert impl._reduce_groups([2, 4, 10], None) == [[0, 1, 2]]


def test_program_tracing_builds_library_nodes():
    @donnx.program
    def conv(X_: (np.float32, (8, 1, 32, 32)), W_: (np.float32, (8, 1, 3, 3)), B_: (np.float32, (8, )),
             Z_: (np.float32, (8, 8, 30, 30))):
        donnx.ONNXConv(X=X_, W=W_, B=B_, Y=Z_)

    g = conv.to_sdfg()
    nodes = [n for n, _ in g.all_nodes_recursive() if isinstance(n, donnx.ONNXOp)]
    assert len(nodes) == 1 and type(nodes[0]).__name__ == "ONNXConv"
    g.expand_library_nodes()
    assert any(isinstance(n, KernelTasklet) for n, _ in g.all_nodes_recursive())


def test_exported_graphs_expand_completely():
    gen = torch.Generator().manual_seed(0)

    def rn(*s):
        return torch.randn(*s, generator=gen) * 0.02

    H, F_ = 128, 256
    p = dict(wq=rn(H, H), bq=rn(H), wk=rn(H, H), bk=rn(H), wv=rn(H, H), bv=rn(H), wo=rn(H, H), bo=rn(H), ln1_g=torch.ones(H),
             ln1_b=torch.zeros(H), w1=rn(F_, H), b1=rn(F_), w2=rn(H, F_), b2=rn(H), ln2_g=torch.ones(H), ln2_b=torch.zeros(H))
    fused = graphs.bert_layer_sdfg(p, 2, 128, 2, fused=True)
    fused.expand_library_nodes()
    order = fused.states()[0].topological_compute_nodes()
    assert [k for t in order for k in t.kernels] == ["gemm", "attention", "gemm", "layernorm", "gemm", "gemm", "layernorm"]
    wide = {k: (v if v.dim() == 1 else v) for k, v in p.items()}
    H2 = 256
    p2 = dict(wq=rn(H2, H2), bq=rn(H2), wk=rn(H2, H2), bk=rn(H2), wv=rn(H2, H2), bv=rn(H2), wo=rn(H2, H2), bo=rn(H2),
              ln1_g=torch.ones(H2), ln1_b=torch.zeros(H2), w1=rn(512, H2), b1=rn(512), w2=rn(H2, 512), b2=rn(H2),
              ln2_g=torch.ones(H2), ln2_b=torch.zeros(H2))
    f2 = graphs.bert_layer_sdfg(p2, 2, 128, 4, fused=True)
    f2.expand_library_nodes()
    # a hidden size the fused kernel covers: LayerNorm rides in the GEMM epilogue, five launches per layer
    assert [k for t in f2.states()[0].topological_compute_nodes() for k in t.kernels] == [
        "gemm", "attention", "gemm_layernorm", "gemm", "gemm_layernorm"]
    unfused = graphs.bert_layer_sdfg(p, 2, 128, 2, fused=False)
    n_nodes = len([n for n, _ in unfused.all_nodes_recursive() if isinstance(n, donnx.ONNXOp)])
    assert n_nodes == 56  # the exported graph: LayerNorm and GELU decomposed, weights as Transpose -> MatMul -> Add
    unfused.expand_library_nodes()
    assert all(isinstance(t, KernelTasklet) for t in unfused.states()[0].topological_compute_nodes())


def test_topological_order_detects_cycles():
    g = sd.SDFG("cyc")
    st = g.add_state()
    g.add_array("a", (4, ), np.float32)
    g.add_array("b", (4, ), np.float32)
    n1, n2 = donnx.ONNXRelu("r1"), donnx.ONNXRelu("r2")
    st.add_edge(st.add_access("a"), None, n1, "X", g.make_array_memlet("a"))
    st.add_edge(n1, "Y", st.add_access("b"), None, g.make_array_memlet("b"))
    st.add_edge(st.add_access("b"), None, n2, "X", g.make_array_memlet("b"))
    st.add_edge(n2, "Y", st.add_access("a"), None, g.make_array_memlet("a"))
    with pytest.raises(ValueError, match="cycle"):
        st.topological_compute_nodes()


def test_validate_checks_the_schema_type_constraints():
    """daceml/onnx/nodes/onnx_op.py:355-417: connectors sharing a type parameter must agree, and the element type must be
    one the parameter allows; a wrong tensor type is a validation error, not "cannot be applied"."""
    import torch
    from daceml_b200 import sdfg as sd

    def one_node(op, ins, outs, **attrs):
        g = sd.SDFG("v")
        st = g.add_state()
        node = getattr(donnx, "ONNX" + op)(op, **attrs)
        st.add_node(node)
        for conn, (shape, dtype) in ins.items():
            g.add_array("i_" + conn, shape, dtype)
            st.add_edge(st.add_read("i_" + conn), None, node, conn, g.make_array_memlet("i_" + conn))
        for conn, (shape, dtype) in outs.items():
            g.add_array("o_" + conn, shape, dtype)
            st.add_edge(node, conn, st.add_write("o_" + conn), None, g.make_array_memlet("o_" + conn))
        return node, g, st

    node, g, st = one_node("MatMul", {"A": ((2, 4), torch.float32), "B": ((4, 3), torch.float16)}, {"Y": ((2, 3), torch.float32)})
    with pytest.raises(ValueError, match="Could not solve type constraints"):
        node.validate(g, st)
    node, g, st = one_node("Softmax", {"input": ((2, 4), torch.int64)}, {"output": ((2, 4), torch.int64)})
    with pytest.raises(ValueError, match="Expected type in"):
        node.validate(g, st)
    node, g, st = one_node("Gather", {"data": ((5, 4), torch.float32), "indices": ((3, ), torch.float32)}, {"output": ((3, 4), torch.float32)})
    with pytest.raises(ValueError, match="for input 'indices'"):
        node.validate(g, st)
    node, g, st = one_node("Where", {"condition": ((4, ), torch.float32), "X": ((4, ), torch.float32), "Y": ((4, ), torch.float32)},
                           {"output": ((4, ), torch.float32)})
    with pytest.raises(ValueError, match="for input 'condition'"):
        node.validate(g, st)
    node, g, st = one_node("Cast", {"input": ((4, ), torch.float32)}, {"output": ((4, ), torch.int64)})
    with pytest.raises(ValueError, match="required attribute 'to'"):
        node.validate(g, st)
    # well-typed nodes pass: mixed types where the schema has separate parameters
    one = one_node("Cast", {"input": ((4, ), torch.float32)}, {"output": ((4, ), torch.int64)}, to=7)
    one[0].validate(one[1], one[2])
    one = one_node("Gather", {"data": ((5, 4), torch.float16), "indices": ((3, ), torch.int64)}, {"output": ((3, 4), torch.float16)})
    one[0].validate(one[1], one[2])


def test_helper_api_for_python_implementations():
    """``python_pure_op_implementation`` / ``program_for_node`` / ``empty_sdfg_for_node``
    (daceml/onnx/op_implementations/utils.py:43-225): registration under the function's name, compute variables,
    the reference's messages for parameters that are not connectors."""
    import torch
    import daceml_b200.onnx as donnx
    from daceml_b200 import sdfg as sd
    from daceml_b200.onnx.forward_implementation_abc import ONNXForward
    from daceml_b200.onnx.op_implementations.utils import (empty_sdfg_for_node, parse_variadic_param, program_for_node,
                                                           python_pure_op_implementation)

    @python_pure_op_implementation(alpha=lambda node: node.alpha, shape=lambda X: X.shape)
    def LeakyRelu(X, Y):
        Y[:] = torch.where(X > 0, X, alpha * X).reshape(shape)  # noqa: F821 - alpha and shape come from compute

    try:
        assert "pure" in donnx.ONNXLeakyRelu.implementations
        assert any(args.get("op") == "LeakyRelu" and args.get("name") == "pure" for _, args in ONNXForward.extensions().items())
        g = sd.SDFG("leaky")
        g.add_array("x", (4, 5), torch.float32)
        g.add_array("y", (4, 5), torch.float32)
        st = g.add_state()
        node = donnx.ONNXLeakyRelu("leaky0", alpha=0.25)
        node.implementation = "pure"
        st.add_edge(st.add_read("x"), None, node, "X", g.make_array_memlet("x"))
        st.add_edge(node, "Y", st.add_write("y"), None, g.make_array_memlet("y"))
        ns, nst, ins, outs = empty_sdfg_for_node(g, st, node)
        assert set(ns.arrays) == {"X", "Y"} and ns.arrays["X"].shape == (4, 5) and not ns.arrays["Y"].transient
        assert set(ins) == {"X"} and set(outs) == {"Y"}
        g.expand_library_nodes()
        (tasklet, ) = [n for n in st.nodes() if isinstance(n, sd.KernelTasklet)]
        x = torch.linspace(-2, 2, 20).reshape(4, 5)
        y = torch.empty(4, 5)
        tasklet.fn({"X": x}, {"Y": y})  # the function itself runs anywhere; compiled SDFGs bind device tensors
        assert torch.equal(y, torch.where(x > 0, x, 0.25 * x))

        def wrong(X, Z):
            pass

        with pytest.raises(ValueError, match="'Z' was not found as an input or output for LeakyRelu"):
            program_for_node(wrong, g, st, node)
        assert parse_variadic_param("Inputs__3") == ("Inputs", 3)
        with pytest.raises(ValueError):
            parse_variadic_param("Inputs__03")
    finally:
        donnx.ONNXLeakyRelu.implementations.pop("pure", None)
        ONNXForward.unregister(LeakyRelu)
