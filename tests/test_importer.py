"""The importer and the module wrapper, as far as they go without a GPU: export, SDFG construction, constant folding,
fusion of real exported graphs, argument checking, hooks."""
import warnings

import pytest
import torch
import torch.nn as nn

import daceml_b200.onnx as donnx
from daceml_b200.onnx.converters import clean_onnx_name
from daceml_b200.onnx.exported_graph import ExportedGraph, GraphNode, ValueInfo, export_module
from daceml_b200.onnx.onnx_importer import ONNXModel
from daceml_b200.torch import DaceModule, dace_module
from daceml_b200.transformation.constant_folding import fold_constants
from models import LeNet, MLP, MBConv, bert_layer

warnings.filterwarnings("ignore")


def test_clean_onnx_name():
    assert clean_onnx_name("onnx::MatMul_12") == "onnxCOLONCOLONMatMul_12"
    assert clean_onnx_name("attention.self.query.bias") == "attentionDOTselfDOTqueryDOTbias"
    assert clean_onnx_name("12") == "ONNX_12"
    assert clean_onnx_name("a/b-c") == "aSLASHbDASHc"


def test_bert_layer_export_imports_node_for_node_and_collapses():
    layer = bert_layer(256, 4, 512).half()
    graph = export_module(layer, (torch.randn(2, 128, 256).half(), ))
    assert [v.name for v in graph.inputs] == ["onnx::MatMul_0"] and graph.inputs[0].shape == (2, 128, 256)
    model = ONNXModel("bert", graph)
    assert model.outputs == ["__return"] and model.sdfg.arg_names == ["onnxCOLONCOLONMatMul_0"]
    ops = [type(n).schema.name for n in model.state.topological_compute_nodes()]
    assert ops.count("MatMul") == 8 and ops.count("Softmax") == 1 and ops.count("Erf") == 1 and ops.count("ReduceMean") == 4
    assert "attention.self.query.bias" in model.weights and "attentionDOTselfDOTqueryDOTbias" in model.clean_weights
    # every parameter of the module is a weight of the model (the exporter renames the pre-transposed matrices)
    assert sum(w.numel() for w in model.weights.values() if w.is_floating_point() and w.dim() > 0) >= sum(
        p.numel() for p in layer.parameters())
    model.auto_optimize()
    assert model.compile_and_init().kernel_names() == ["gemm", "attention", "gemm_layernorm", "gemm", "gemm_layernorm"]
    att = next(n for n in model.state.nodes() if type(n).__name__ == "KernelTasklet" and n.kernels == ("attention", ))
    assert att is not None


def test_attention_fusion_only_where_the_kernel_applies():
    """fp32 layers and head sizes other than 64 keep MatMul / Softmax / MatMul instead of failing at expansion."""
    for layer, x in ((bert_layer(256, 4, 512), torch.randn(2, 128, 256)), (bert_layer(96, 4, 128).half(), torch.randn(2, 16, 96).half())):
        names = DaceModule(layer, dummy_inputs=(x, )).compiled_function.kernel_names()
        assert "attention" not in names and names.count("softmax") == 1 and names.count("gemm") == 8


def test_daceml_module_wraps_the_benchmark_modules():
    m = DaceModule(MLP(), dummy_inputs=(torch.randn(64, 784), ))
    assert m.compiled_function.kernel_names() == ["gemm", "gemm", "gemm", "softmax"]
    m = DaceModule(MBConv(), dummy_inputs=(torch.randn(2, 24, 8, 8), ))
    assert m.compiled_function.kernel_names() == ["conv2d", "conv2d", "se_gate", "conv2d"]
    m = DaceModule(nn.Conv2d(3, 16, 3, stride=2, bias=False), dummy_inputs=(torch.randn(2, 3, 16, 16), ))
    assert m.compiled_function.kernel_names() == ["conv2d"]
    assert m.sdfg is m.dace_model.sdfg and m.sdfg.name == "Conv2d"
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            m(torch.randn(2, 3, 16, 16))


def test_module_argument_checks_and_hooks():
    with pytest.raises(NotImplementedError):
        DaceModule(MLP(), backward=True)
    with pytest.raises(NotImplementedError):
        DaceModule(MLP(), training=True)
    with pytest.raises(ValueError):
        DaceModule(MLP(), cuda=False)
    order = []
    m = DaceModule(MLP(), auto_optimize=False)
    m.append_post_onnx_hook("second", lambda mod: order.append(("second", len(mod.sdfg.states()[0].nodes()))))
    m.prepend_post_onnx_hook("first", lambda mod: order.append(("first", type(mod.dace_model).__name__)))
    m.append_post_onnx_hook("second", lambda mod: order.append(("second_again", None)))  # renamed, not replaced
    m.append_post_compile_hook("compiled", lambda c: order.append(("compiled", c.kernel_names())))
    assert list(m.post_onnx_hooks) == ["first", "second", "second_0"]
    m.function = m._initialize_sdfg((torch.randn(8, 784), ))
    assert [o[0] for o in order] == ["first", "second", "second_again", "compiled"]
    # without auto_optimize nothing was fused: three Gemm launches, two Relu, one LogSoftmax
    assert order[-1][1] == ["gemm", "unary", "gemm", "unary", "gemm", "softmax"]
    m.reset_sdfg()
    assert m.function is None
    with pytest.raises(NotImplementedError):
        m.train()

    @dace_module(sdfg_name="decorated")
    class Decorated(nn.Module):
        def forward(self, x):
            return torch.sqrt(torch.log(x))

    d = Decorated()
    assert isinstance(d, DaceModule) and d.sdfg_name == "decorated"


def test_module_is_registered_as_a_torch_operator():
    """``compile_torch_extension`` (default): ``torch.ops.daceml_<name>.<name>(handle, *inputs)`` with a schema and a
    shape function, as the reference's generated extension declares it (cpp_torch_extension.py:398-457)."""
    m = DaceModule(MLP(), dummy_inputs=(torch.randn(16, 784), ), sdfg_name="mlp_as_op")
    assert m.torch_op is torch.ops.daceml_mlp_as_op.mlp_as_op
    assert str(m.torch_op.default._schema) == "daceml_mlp_as_op::mlp_as_op(int handle_ptr, Tensor onnxCOLONCOLONGemm_0) -> Tensor"
    out = m.torch_op(m.torch_op_handle, torch.empty(16, 784, device="meta"))
    assert out.shape == (16, 10) and out.dtype == torch.float32 and out.device.type == "meta"
    again = DaceModule(MLP(), dummy_inputs=(torch.randn(16, 784), ), sdfg_name="mlp_as_op")  # same name: numbered namespace
    assert again.torch_op is torch.ops.daceml_mlp_as_op_1.mlp_as_op
    plain = DaceModule(MLP(), dummy_inputs=(torch.randn(16, 784), ), compile_torch_extension=False)
    assert plain.torch_op is None

    class Two(nn.Module):
        def forward(self, x, y):
            return x + y, x * y

    two = DaceModule(Two(), dummy_inputs=(torch.randn(4), torch.randn(4)), sdfg_name="two_outputs_op")
    assert str(two.torch_op.default._schema).endswith("-> Tensor[]")
    a, b = two.torch_op(two.torch_op_handle, torch.empty(4, device="meta"), torch.empty(4, device="meta"))
    assert a.shape == b.shape == (4, )


def test_parameter_to_transient_is_accepted():
    """tests/torch/test_bert_encoder.py:26-31 registers this as a post-ONNX hook for every parameter on the GPU."""
    from daceml_b200.transformation import parameter_to_transient
    m = DaceModule(MLP())

    def param_to_trans(model):
        for name, _ in model.model.named_parameters():
            parameter_to_transient(model, name)

    m.append_post_onnx_hook("param_to_transient", param_to_trans)
    m.function = m._initialize_sdfg((torch.randn(8, 784), ))
    assert m.compiled_function.kernel_names() == ["gemm", "gemm", "gemm", "softmax"]
    with pytest.raises(AttributeError):
        parameter_to_transient(m, "no.such.weight")


def test_debug_transients_become_outputs():
    m = DaceModule(MLP(), dummy_inputs=(torch.randn(8, 784), ), auto_optimize=False, debug_transients=True)
    assert len(m.dace_model.outputs) == 6 and not any(d.transient for d in m.sdfg.arrays.values())


def test_reshapes_become_views():
    """After the fusion pass a Reshape into a transient is a view of its input; one that produces a model output turns
    its input into a view of the output, so the producer writes in place; launch order still follows the data."""
    m = DaceModule(LeNet(), dummy_inputs=(torch.rand(8, 1, 32, 32), ))
    assert m.compiled_function.kernel_names() == ["conv2d", "maxpool2d", "conv2d", "maxpool2d", "gemm", "gemm", "gemm", "softmax"]
    views = {n: d.view_of for n, d in m.sdfg.arrays.items() if d.view_of}
    assert len(views) == 1
    (flat, pooled), = views.items()
    assert m.sdfg.arrays[flat].shape == (8, 576) and m.sdfg.arrays[pooled].shape == (8, 16, 6, 6)
    assert m.sdfg.root_of(flat) == pooled

    class Tail(nn.Module):
        def forward(self, x):
            return torch.relu(x).reshape(4, 6), torch.exp(x).reshape(2, 12).reshape(24)

    m = DaceModule(Tail(), dummy_inputs=(torch.rand(2, 3, 4), ))
    assert m.compiled_function.kernel_names() == ["unary", "unary"]
    assert sorted(m.sdfg.root_of(n) for n, d in m.sdfg.arrays.items() if d.view_of) == ["__return_0", "__return_1"]
    # without the pass every reshape is a copy
    m = DaceModule(Tail(), dummy_inputs=(torch.rand(2, 3, 4), ), auto_optimize=False)
    assert len(m.compiled_function.kernel_names()) == 5


def test_batchnorm_folds_into_conv_or_becomes_one_launch():
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv, self.bn, self.bn2 = nn.Conv2d(3, 8, 3, padding=1, bias=False), nn.BatchNorm2d(8), nn.BatchNorm2d(8)

        def forward(self, x):
            return self.bn2(torch.relu(self.bn(self.conv(x))))

    net = Net().eval()
    graph = export_module(net, (torch.randn(2, 3, 8, 8), ), do_constant_folding=False)  # keeps Conv -> BatchNormalization
    assert [n.op_type for n in graph.nodes] == ["Conv", "BatchNormalization", "Relu", "BatchNormalization"]
    model = ONNXModel("bn", graph)
    model.auto_optimize()
    # Conv+BN+Relu is one convolution, the free-standing BN one depthwise launch
    assert model.compile_and_init().kernel_names() == ["conv2d", "conv2d"]
    folded = next(t for n, t in model.sdfg.constants.items() if n.endswith("_w"))
    a = net.bn.weight / torch.sqrt(net.bn.running_var + net.bn.eps)
    assert torch.allclose(folded, net.conv.weight * a.reshape(-1, 1, 1, 1), atol=1e-6)


def _vi(name, shape, dtype=torch.float32):
    return ValueInfo(name, tuple(shape), dtype)


def _shape_chain_graph():
    """x[2,3,4] -> Reshape(x, Concat(Unsqueeze(Gather(Shape(x), 0)), [-1])) -> Relu: what an export without
    exporter-side folding contains for ``x.reshape(x.shape[0], -1)``."""
    infos = {v.name: v for v in [
        _vi("x", (2, 3, 4)), _vi("shp", (3, ), torch.int64), _vi("zero", (), torch.int64), _vi("b", (), torch.int64),
        _vi("b1", (1, ), torch.int64), _vi("minus", (1, ), torch.int64), _vi("target", (2, ), torch.int64), _vi("flat", (2, 12)),
        _vi("y", (2, 12))]}
    nodes = [
        GraphNode("Shape", "shape", ["x"], ["shp"]),
        GraphNode("Constant", "c0", [], ["zero"], dict(value=torch.tensor(0))),
        GraphNode("Gather", "gather", ["shp", "zero"], ["b"], dict(axis=0)),
        GraphNode("Unsqueeze", "unsq", ["b"], ["b1"], dict(axes=[0])),
        GraphNode("Constant", "c1", [], ["minus"], dict(value_ints=[-1])),
        GraphNode("Concat", "cat", ["b1", "minus"], ["target"], dict(axis=0)),
        GraphNode("Reshape", "reshape", ["x", "target"], ["flat"]),
        GraphNode("Relu", "relu", ["flat"], ["y"]),
    ]
    return ExportedGraph([infos["x"]], [infos["y"]], {}, infos, nodes)


def test_constant_folding_removes_shape_arithmetic():
    model = ONNXModel("chain", _shape_chain_graph())
    st = model.state
    assert len(st.topological_compute_nodes()) == 6
    cat = next(n for n in st.nodes() if isinstance(n, donnx.ONNXConcat))
    assert sorted(e.dst_conn for e in st.in_edges(cat)) == ["inputs__0", "inputs__1"]
    assert fold_constants(model.sdfg) == 4
    assert [type(n).schema.name for n in st.topological_compute_nodes()] == ["Reshape", "Relu"]
    assert model.sdfg.constants["target"].tolist() == [2, -1]
    assert "shp" not in model.sdfg.arrays and "b1" not in model.sdfg.arrays
    assert fold_constants(model.sdfg) == 0
    # a weight transpose folds into a new weight
    w = torch.arange(6.0).reshape(2, 3)
    infos = {v.name: v for v in [_vi("x", (4, 3)), _vi("w", (2, 3)), _vi("wt", (3, 2)), _vi("y", (4, 2))]}
    g = ExportedGraph([infos["x"]], [infos["y"]], dict(w=w), infos,
                      [GraphNode("Transpose", "t", ["w"], ["wt"], dict(perm=[1, 0])), GraphNode("MatMul", "mm", ["x", "wt"], ["y"])])
    model = ONNXModel("lin", g)
    model.auto_optimize()
    assert model.compile_and_init().kernel_names() == ["gemm"]
    assert any(torch.equal(c, w) or torch.equal(c, w.t()) for c in model.sdfg.constants.values())


def test_importer_rejects_bad_graphs_and_arguments():
    infos = {v.name: v for v in [_vi("x", (4, )), _vi("y", (4, ))]}
    with pytest.raises(ValueError, match="Unsupported ONNX operator: 'NonMaxSuppression'"):
        ONNXModel("bad", ExportedGraph([infos["x"]], [infos["y"]], {}, infos, [GraphNode("NonMaxSuppression", "n", ["x"], ["y"])]))
    with pytest.raises(ValueError, match="exactly one"):
        ONNXModel("bad", ExportedGraph([infos["x"]], [infos["y"]], {}, infos,
                                       [GraphNode("Constant", "c", [], ["y"], dict(value_int=1, value_float=1.0))]))
    with pytest.raises(ValueError, match="Could not find array"):
        ONNXModel("bad", ExportedGraph([infos["x"]], [infos["y"]], {}, infos, [GraphNode("Relu", "r", ["ghost"], ["y"])]))
    with pytest.raises(ValueError, match="no CPU path"):
        ONNXModel("bad", ExportedGraph([infos["x"]], [infos["y"]], {}, infos, [GraphNode("Relu", "r", ["x"], ["y"])]), cuda=False)
    model = ONNXModel("ok", ExportedGraph([infos["x"]], [infos["y"]], {}, infos, [GraphNode("Relu", "r", ["x"], ["y"])]))
    with pytest.raises(ValueError, match="Expected 1 arguments, got 2"):
        model(torch.zeros(4), torch.zeros(4))
    with pytest.raises(ValueError, match="Missing inputs x"):
        model()
    with pytest.raises(ValueError, match="Unknown inputs z"):
        model(torch.zeros(4), z=torch.zeros(4))
    # an optional input that is left out keeps its connector free (Clip without min)
    infos2 = dict(infos, hi=_vi("hi", ()))
    g = ExportedGraph([infos["x"]], [infos["y"]], dict(hi=torch.tensor(1.0)), infos2, [GraphNode("Clip", "clip", ["x", None, "hi"], ["y"])])
    clip = ONNXModel("clip", g)
    node = clip.state.topological_compute_nodes()[0]
    assert sorted(e.dst_conn for e in clip.state.in_edges(node)) == ["input", "max"]


def test_model_proto_route_needs_onnx():
    onnx = pytest.importorskip("onnx")
    from onnx import helper, TensorProto
    node = helper.make_node("Relu", ["x"], ["y"])
    graph = helper.make_graph([node], "g", [helper.make_tensor_value_info("x", TensorProto.FLOAT, [4])],
                              [helper.make_tensor_value_info("y", TensorProto.FLOAT, [4])])
    model = ONNXModel("proto", helper.make_model(graph, opset_imports=[helper.make_opsetid("", 12)]))
    assert [type(n).schema.name for n in model.state.topological_compute_nodes()] == ["Relu"]


def test_resnet_basic_block_collapses_to_two_convolutions_and_a_relu():
    """Conv + BatchNorm (+ ReLU) fold into one convolution each, the shortcut add rides in the second one's epilogue;
    the down-sampling block has a third convolution (strided 1x1 + BatchNorm) for the shortcut."""
    class BasicBlock(nn.Module):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.conv1, self.bn1 = nn.Conv2d(cin, cout, 3, stride=stride, padding=1, bias=False), nn.BatchNorm2d(cout)
            self.conv2, self.bn2 = nn.Conv2d(cout, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

        def forward(self, x):
            y = torch.relu(self.bn1(self.conv1(x)))
            y = self.bn2(self.conv2(y))
            return torch.relu(y + (x if self.down is None else self.down(x)))

    m = DaceModule(BasicBlock(16, 16, 1).eval(), dummy_inputs=(torch.randn(2, 16, 12, 12), ))
    assert m.compiled_function.kernel_names() == ["conv2d", "conv2d", "unary"]
    fused = [n for n, _ in m.sdfg.all_nodes_recursive() if type(n).__name__ == "KernelTasklet"]
    assert len(fused) == 3
    m = DaceModule(BasicBlock(16, 32, 2).eval(), dummy_inputs=(torch.randn(2, 16, 12, 12), ))
    assert sorted(m.compiled_function.kernel_names()) == ["conv2d", "conv2d", "conv2d", "unary"]
