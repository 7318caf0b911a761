"""An ONNX graph held in plain Python objects, and the two ways to obtain one.

The reference reads ``onnx.ModelProto`` files written by ``torch.onnx.export(..., opset_version=12)``
(``daceml/torch/module.py:269-291``, ``daceml/onnx/onnx_importer.py:117-205``).  The ``onnx`` package
is optional for this library, so the importer works on :class:`ExportedGraph`, which is filled

* from an ``nn.Module`` by the TorchScript exporter's graph pass (:func:`export_module`) - the same
  opset-12 conversion ``torch.onnx.export`` runs, stopped before protobuf serialisation; or
* from a ``ModelProto`` (:func:`from_model_proto`), when ``onnx`` can be imported.
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .converters import onnx_tensor_type_to_torch


@dataclass
class ValueInfo:
    name: str
    shape: Optional[Tuple[int, ...]]
    dtype: Optional[torch.dtype]


@dataclass
class GraphNode:
    op_type: str
    name: str
    inputs: List[Optional[str]]  # None marks an omitted optional input
    outputs: List[str]
    attributes: Dict[str, object] = field(default_factory=dict)


@dataclass
class ExportedGraph:
    inputs: List[ValueInfo]
    outputs: List[ValueInfo]
    initializers: Dict[str, torch.Tensor]
    value_infos: Dict[str, ValueInfo]
    nodes: List[GraphNode]
    opset: int = 12


# ---------------------------------------------------------------------------------------------
# nn.Module -> ExportedGraph
# ---------------------------------------------------------------------------------------------
def _value_info(v) -> ValueInfo:
    t = v.type()
    shape = dtype = None
    if isinstance(t, torch._C.TensorType):
        sizes = t.sizes()
        shape = tuple(int(s) for s in sizes) if sizes is not None else None
        dtype = t.dtype()
    return ValueInfo(v.debugName(), shape, dtype)


def _attribute(node, key):
    kind = node.kindOf(key)
    if kind == "t":
        return node.t(key)
    if kind in ("i", "f", "s"):
        return getattr(node, kind)(key)
    if kind in ("is", "fs", "ss"):
        return list(getattr(node, kind)(key))
    raise NotImplementedError("attribute '{}' of kind '{}' on {}".format(key, kind, node.kind()))


def export_module(module: torch.nn.Module, dummy_inputs, training: bool = False, do_constant_folding: bool = True,
                  opset_version: int = 12) -> ExportedGraph:
    """Traces ``module`` on ``dummy_inputs`` and converts the trace to ONNX operators at ``opset_version``.

    With ``do_constant_folding`` the exporter folds the weight transposes of ``nn.Linear`` and every shape
    computation of a statically shaped trace (the job onnx-simplifier does for the reference,
    ``onnx_importer.py:60-67``).  Parameters end up in ``initializers``; only the traced tensors are ``inputs``.
    """
    try:
        from torch.onnx._internal.torchscript_exporter import utils as ts_utils
        from torch.onnx._internal.torchscript_exporter._globals import GLOBALS
    except ImportError as e:  # pragma: no cover - depends on the torch build
        raise RuntimeError("this torch build has no TorchScript ONNX exporter; pass an ExportedGraph or a ModelProto") from e
    if training:
        raise NotImplementedError("only inference graphs are imported (BatchNorm statistics and Dropout masks are "
                                  "training-mode state this library has no kernels for)")
    if not isinstance(dummy_inputs, (tuple, list)):
        dummy_inputs = (dummy_inputs, )
    previous = GLOBALS.export_onnx_opset_version
    was_training = module.training
    GLOBALS.export_onnx_opset_version = opset_version
    try:
        module.eval()
        with torch.no_grad():
            graph, params, _ = ts_utils._model_to_graph(module, tuple(dummy_inputs), do_constant_folding=do_constant_folding)
    finally:
        GLOBALS.export_onnx_opset_version = previous
        module.train(was_training)

    initializers = {k: v.detach() for k, v in params.items()}
    value_infos: Dict[str, ValueInfo] = {}
    inputs = []
    for v in graph.inputs():
        vi = _value_info(v)
        value_infos[vi.name] = vi
        if vi.name not in initializers:
            inputs.append(vi)
    nodes = []
    for i, n in enumerate(graph.nodes()):
        kind = n.kind()
        if kind == "prim::Constant":  # an omitted optional input
            continue
        if not kind.startswith("onnx::"):
            raise ValueError("Unsupported operator in the exported graph: '{}'".format(kind))
        ins = [None if (v.node().kind() == "prim::Constant" and v.node().mustBeNone()) else v.debugName() for v in n.inputs()]
        while ins and ins[-1] is None:
            ins.pop()
        outs = []
        for v in n.outputs():
            vi = _value_info(v)
            value_infos[vi.name] = vi
            outs.append(vi.name)
        attrs = {k: _attribute(n, k) for k in n.attributeNames()}
        nodes.append(GraphNode(kind[len("onnx::"):], "{}_{}".format(kind[len("onnx::"):], i), ins, outs, attrs))
    outputs = [value_infos.get(v.debugName()) or _value_info(v) for v in graph.outputs()]
    return ExportedGraph(inputs, outputs, initializers, value_infos, nodes, opset_version)


# ---------------------------------------------------------------------------------------------
# onnx.ModelProto -> ExportedGraph
# ---------------------------------------------------------------------------------------------
def _proto_value_info(value) -> ValueInfo:
    tt = value.type.tensor_type
    shape = None
    if tt.HasField("shape"):
        dims = []
        for d in tt.shape.dim:
            if not d.HasField("dim_value"):
                raise NotImplementedError("value '{}' has a symbolic dimension; export with static shapes".format(value.name))
            dims.append(int(d.dim_value))
        shape = tuple(dims)
    return ValueInfo(value.name, shape, onnx_tensor_type_to_torch(tt.elem_type))


def from_model_proto(model) -> ExportedGraph:
    """Converts a checked, shape-inferred ``onnx.ModelProto`` (what ``onnx_importer.py:117-126`` prepares)."""
    import onnx
    from onnx import numpy_helper, shape_inference
    onnx.checker.check_model(model)
    model = shape_inference.infer_shapes(model)
    g = model.graph
    opset = next((o.version for o in model.opset_import if o.domain == ""), 12)
    initializers = {t.name: torch.from_numpy(numpy_helper.to_array(t).copy()) for t in g.initializer}
    value_infos = {v.name: _proto_value_info(v) for v in list(g.input) + list(g.output) + list(g.value_info)}
    inputs = [value_infos[v.name] for v in g.input if v.name not in initializers]
    outputs = [value_infos[v.name] for v in g.output]
    nodes = []
    for i, n in enumerate(g.node):
        attrs = {}
        for a in n.attribute:
            val = onnx.helper.get_attribute_value(a)
            if a.type == onnx.AttributeProto.TENSOR:
                val = torch.from_numpy(numpy_helper.to_array(val).copy())
            elif a.type == onnx.AttributeProto.STRING:
                val = val.decode("utf-8")
            elif a.type in (onnx.AttributeProto.INTS, onnx.AttributeProto.FLOATS):
                val = list(val)
            attrs[a.name] = val
        ins = [name if name else None for name in n.input]
        nodes.append(GraphNode(n.op_type, n.name or "{}_{}".format(n.op_type, i), ins, list(n.output), attrs))
    return ExportedGraph(inputs, outputs, initializers, value_infos, nodes, opset)
