"""Operator schemas for the ONNX opset-12 operators on the hot path.

The reference mirrors ``onnx.defs`` schemas at import time (``daceml/onnx/schema.py``,
``daceml/onnx/nodes/onnx_op.py:510-556``).  The ``onnx`` package is not a dependency here, so the
connector names, their kinds and the attribute defaults of the operators this library implements
are written out; they are the names an expansion sees (``A, B, Y``; ``X, W, B, Y``;
``Inputs__0 ...``, ``Output``; ``data, reduced``).

Four fused operators that opset 12 does not have (``LayerNormalization`` and ``Gelu`` exist in
later opsets; ``FusedMatMul`` and ``Attention`` are the usual contrib names) are declared with
``fused=True``: they are what the fusion pass rewrites exported sub-graphs into.
"""
from collections import namedtuple

import torch

SINGLE, OPTIONAL, VARIADIC = "single", "optional", "variadic"

# type constraints, as ONNX schemas state them (``tensor(float)`` ... by type parameter): every connector has a type
# parameter ("T" unless said otherwise); connectors with the same parameter must carry the same element type, and the
# type must be one the parameter allows
FLOATS = (torch.float16, torch.float32, torch.float64)
INTS = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)
NUMERIC = FLOATS + INTS
ANY = NUMERIC + (torch.bool, )
INDEX = (torch.int32, torch.int64)
_FLOAT_ONLY = {"Softmax", "LogSoftmax", "Sqrt", "Sigmoid", "Reciprocal", "Softplus", "LeakyRelu", "Erf", "Exp", "Log", "Tanh",
               "Gemm", "Conv", "GlobalAveragePool", "BatchNormalization", "MaxPool", "LayerNormalization", "Gelu", "Swish",
               "FusedMatMul", "Attention", "FusedConv", "SqueezeExcite", "ReduceMean", "Clip", "Relu", "Einsum"}
# connector -> type parameter, where it is not "T"; type parameter -> allowed types, where it is not the operator default
_TYPE_PARAMS = {
    "Cast": ({"input": "T1", "output": "T2"}, {"T1": ANY, "T2": ANY}),
    "Gather": ({"indices": "Tind"}, {"T": ANY, "Tind": INDEX}),
    "Shape": ({"shape": "T1"}, {"T": ANY, "T1": (torch.int64, )}),
    "Reshape": ({"shape": "Tshape"}, {"T": ANY, "Tshape": (torch.int64, )}),
    "Expand": ({"shape": "Tshape"}, {"T": ANY, "Tshape": (torch.int64, )}),
    "Slice": ({"starts": "Tind", "ends": "Tind", "axes": "Tind", "steps": "Tind"}, {"T": ANY, "Tind": INDEX}),
    "Where": ({"condition": "B"}, {"T": ANY, "B": (torch.bool, )}),
    "MaxPool": ({"Indices": "I"}, {"I": (torch.int64, )}),
    "ConstantOfShape": ({"input": "T1", "output": "T2"}, {"T1": (torch.int64, ), "T2": ANY}),
}
_TYPE_PARAMS["Pow"] = ({"Y": "T1"}, {"T1": NUMERIC})
_TYPE_PARAMS["LayerNormalization"] = ({"Scale": "U", "B": "U"}, {"U": FLOATS})
_TYPE_PARAMS["FusedMatMul"] = ({"LnScale": "U", "LnBias": "U"}, {"U": FLOATS})
for _cmp in ("Equal", "Greater", "Less", "GreaterOrEqual", "LessOrEqual"):
    _TYPE_PARAMS[_cmp] = ({"C": "T1"}, {"T": ANY if _cmp == "Equal" else NUMERIC, "T1": (torch.bool, )})
for _move in ("Identity", "Transpose", "Flatten", "Unsqueeze", "Squeeze", "Concat", "Split"):
    _TYPE_PARAMS[_move] = ({}, {"T": ANY})
_REQUIRED_ATTRIBUTES = {"Einsum": ("equation", ), "Cast": ("to", )}

Param = namedtuple("Param", ["name", "kind"])


class ONNXSchema:
    def __init__(self, name, inputs, outputs, attributes=None, fused=False, host_only=False, doc=""):
        self.name = name
        self.inputs = [Param(*p) if isinstance(p, tuple) else Param(p, SINGLE) for p in inputs]
        self.outputs = [Param(*p) if isinstance(p, tuple) else Param(p, SINGLE) for p in outputs]
        self.attributes = dict(attributes or {})
        self.fused = fused
        self.host_only = host_only
        self.doc = doc
        params, allowed = _TYPE_PARAMS.get(name, ({}, {}))
        self.type_params = {p.name: params.get(p.name, "T") for p in self.inputs + self.outputs}
        self.type_constraints = {"T": FLOATS if name in _FLOAT_ONLY else NUMERIC}
        self.type_constraints.update(allowed)
        self.required_attributes = _REQUIRED_ATTRIBUTES.get(name, ())

    def non_variadic_inputs(self):
        return [p.name for p in self.inputs if p.kind != VARIADIC]

    def variadic_inputs(self):
        return [p.name for p in self.inputs if p.kind == VARIADIC]

    def non_variadic_outputs(self):
        return [p.name for p in self.outputs if p.kind != VARIADIC]

    def variadic_outputs(self):
        return [p.name for p in self.outputs if p.kind == VARIADIC]


def _unary(name, i="X", o="Y", **attrs):
    return ONNXSchema(name, [i], [o], attrs)


_S = [
    ONNXSchema("MatMul", ["A", "B"], ["Y"]),
    ONNXSchema("Gemm", ["A", "B", ("C", OPTIONAL)], ["Y"], dict(alpha=1.0, beta=1.0, transA=0, transB=0)),
    ONNXSchema("Einsum", [("Inputs", VARIADIC)], ["Output"], dict(equation=None)),
    ONNXSchema("Softmax", ["input"], ["output"], dict(axis=1)),
    ONNXSchema("LogSoftmax", ["input"], ["output"], dict(axis=1)),
    ONNXSchema("Add", ["A", "B"], ["C"]),
    ONNXSchema("Sub", ["A", "B"], ["C"]),
    ONNXSchema("Mul", ["A", "B"], ["C"]),
    ONNXSchema("Div", ["A", "B"], ["C"]),
    ONNXSchema("Pow", ["X", "Y"], ["Z"]),
    _unary("Sqrt"), _unary("Relu"), _unary("Sigmoid"), _unary("Reciprocal"), _unary("Softplus"),
    _unary("LeakyRelu", alpha=0.01),
    _unary("Erf", "input", "output"), _unary("Exp", "input", "output"), _unary("Log", "input", "output"),
    _unary("Tanh", "input", "output"), _unary("Identity", "input", "output"),
    ONNXSchema("Clip", ["input", ("min", OPTIONAL), ("max", OPTIONAL)], ["output"]),
    ONNXSchema("Cast", ["input"], ["output"], dict(to=None)),
    ONNXSchema("ReduceMean", ["data"], ["reduced"], dict(axes=None, keepdims=1)),
    ONNXSchema("ReduceSum", ["data"], ["reduced"], dict(axes=None, keepdims=1)),
    ONNXSchema("ReduceMax", ["data"], ["reduced"], dict(axes=None, keepdims=1)),
    ONNXSchema("ReduceMin", ["data"], ["reduced"], dict(axes=None, keepdims=1)),
    ONNXSchema("Transpose", ["data"], ["transposed"], dict(perm=None)),
    ONNXSchema("Reshape", ["data", ("shape", OPTIONAL)], ["reshaped"]),
    ONNXSchema("Flatten", ["input"], ["output"], dict(axis=1)),
    ONNXSchema("Unsqueeze", ["data"], ["expanded"], dict(axes=None)),
    ONNXSchema("Squeeze", ["data"], ["squeezed"], dict(axes=None)),
    ONNXSchema("Sum", [("data_0", VARIADIC)], ["sum"]),
    ONNXSchema("Conv", ["X", "W", ("B", OPTIONAL)], ["Y"],
               dict(auto_pad="NOTSET", dilations=None, group=1, kernel_shape=None, pads=None, strides=None)),
    ONNXSchema("GlobalAveragePool", ["X"], ["Y"]),
    # inference form only: Y from the running statistics (the training-mode outputs have no kernel here)
    ONNXSchema("BatchNormalization", ["X", "scale", "B", "mean", "var"], ["Y"], dict(epsilon=1e-5, momentum=0.9)),
    # data movement (one strided-copy / gather kernel each; on constant inputs they fold at build time)
    ONNXSchema("Shape", ["data"], ["shape"]),
    ONNXSchema("Gather", ["data", "indices"], ["output"], dict(axis=0)),
    ONNXSchema("Concat", [("inputs", VARIADIC)], ["concat_result"], dict(axis=None)),
    ONNXSchema("Slice", ["data", "starts", "ends", ("axes", OPTIONAL), ("steps", OPTIONAL)], ["output"]),
    ONNXSchema("Split", ["input"], [("outputs", VARIADIC)], dict(axis=0, split=None)),
    ONNXSchema("Expand", ["input", "shape"], ["output"]),
    ONNXSchema("Where", ["condition", "X", "Y"], ["output"]),
    ONNXSchema("MaxPool", ["X"], ["Y", ("Indices", OPTIONAL)],
               dict(auto_pad="NOTSET", ceil_mode=0, dilations=None, kernel_shape=None, pads=None, storage_order=0, strides=None)),
    _unary("Neg"),
    ONNXSchema("Equal", ["A", "B"], ["C"]), ONNXSchema("Greater", ["A", "B"], ["C"]), ONNXSchema("Less", ["A", "B"], ["C"]),
    ONNXSchema("GreaterOrEqual", ["A", "B"], ["C"]), ONNXSchema("LessOrEqual", ["A", "B"], ["C"]),
    # only ever evaluated on the host by the constant-folding pass (its input is a shape)
    ONNXSchema("ConstantOfShape", ["input"], ["output"], dict(value=None), host_only=True),
    # fused operators (targets of the fusion pass)
    ONNXSchema("LayerNormalization", ["X", ("Scale", OPTIONAL), ("B", OPTIONAL), ("Residual", OPTIONAL)], ["Y"],
               dict(axis=-1, epsilon=1e-5), fused=True),
    ONNXSchema("Gelu", ["X"], ["Y"], fused=True),
    ONNXSchema("Swish", ["X"], ["Y"], fused=True),
    ONNXSchema("FusedMatMul", ["A", "B", ("Bias", OPTIONAL), ("Residual", OPTIONAL), ("LnScale", OPTIONAL),
                               ("LnBias", OPTIONAL)], ["Y"],
               dict(alpha=1.0, transB=0, activation="", ln_epsilon=None), fused=True),
    ONNXSchema("Attention", ["Q", ("K", OPTIONAL), ("V", OPTIONAL), ("Mask", OPTIONAL)], ["Y"], dict(num_heads=1, scale=None), fused=True),
    ONNXSchema("FusedConv", ["X", "W", ("B", OPTIONAL), ("Gate", OPTIONAL), ("Residual", OPTIONAL)],
               ["Y", ("Pool", OPTIONAL)],
               dict(dilations=None, group=1, kernel_shape=None, pads=None, strides=None, activation=""), fused=True),
    ONNXSchema("SqueezeExcite", ["X", "W1", ("B1", OPTIONAL), "W2", ("B2", OPTIONAL)], ["Y"], fused=True),
]

SCHEMAS = {s.name: s for s in _S}
