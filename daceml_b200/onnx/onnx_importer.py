"""Loads an exported ONNX graph into an SDFG of ONNX library nodes.

Mirror of the reference's ``ONNXModel`` (``daceml/onnx/onnx_importer.py:73-338`` builds the SDFG,
``:469-515`` runs it): model inputs and outputs become arrays, initializers and ``Constant`` nodes
become constants held in ``weights``, every other node becomes ``ONNX<op_type>`` wired by the
schema's connector names (variadic parameters as ``name__i``), and the outputs are named
``__return`` / ``__return_i``.  Calling the model optimises (constant folding, fusion, expansion to
kernel launches), compiles once, and runs on the current CUDA stream.
"""
import logging
from typing import Dict, List, Optional

import torch

from daceml_b200 import sdfg as sd
from .converters import clean_onnx_name
from .exported_graph import ExportedGraph, GraphNode, export_module, from_model_proto
from .nodes.onnx_op import get_onnx_node, has_onnx_node
from .schema import VARIADIC

log = logging.getLogger(__name__)

_CONSTANT_ATTRS = ("sparse_value", "value", "value_float", "value_floats", "value_int", "value_ints", "value_string",
                   "value_strings")


def _constant_value(node: GraphNode) -> torch.Tensor:
    """The tensor of a ``Constant`` node, with the reference's checks (``onnx_importer.py:208-233``)."""
    unexpected = set(node.attributes) - set(_CONSTANT_ATTRS)
    if unexpected:
        raise ValueError("Got unexpected attributes on Constant node {}".format(sorted(unexpected)))
    if len(node.attributes) != 1:
        raise ValueError("Expected Constant node to have exactly one of its attributes set")
    if len(node.inputs) != 0 or len(node.outputs) != 1:
        raise ValueError("Expected Constant node to have no inputs and exactly 1 output")
    key, val = next(iter(node.attributes.items()))
    if key == "value":
        return val
    if key == "value_float":
        return torch.tensor(val, dtype=torch.float32)
    if key == "value_floats":
        return torch.tensor(list(val), dtype=torch.float32)
    if key == "value_int":
        return torch.tensor(val, dtype=torch.int64)
    if key == "value_ints":
        return torch.tensor(list(val), dtype=torch.int64)
    raise NotImplementedError("Constant attribute '{}'".format(key))


class ONNXModel:
    """Loads an ONNX model into an SDFG.

    :param name: the name for the SDFG.
    :param model: an :class:`ExportedGraph`, or an ``onnx.ModelProto`` when ``onnx`` is installed.
    :param cuda: must be true (or ``None``): this library has no CPU path.
    :param auto_optimize: fold constants, fuse sub-graphs and expand the nodes before the first call.
    :param save_transients: if not None, the intermediate tensors of each call are stored in this dict
                            (they only exist for nodes the fusion pass left alone).
    ``simplify``, ``onnx_simplify``, ``storage`` and ``auto_merge`` are accepted for signature
    compatibility; shapes are static and simplification is the exporter's and the fusion pass's job.
    """

    def __init__(self, name: str, model, cuda: Optional[bool] = None, auto_optimize: bool = True, simplify: bool = False,
                 onnx_simplify: bool = True, storage=None, save_transients: Optional[Dict[str, torch.Tensor]] = None,
                 auto_merge: bool = False):
        if cuda is not None and not cuda:
            raise ValueError("daceml_b200 has no CPU path: ONNXModel needs cuda=True")
        if not isinstance(model, ExportedGraph):
            model = from_model_proto(model)
        if model.opset != 12:
            log.warning("Expected the onnx model to be exported with opset 12, got %s. This model may fail to import "
                        "as a result.", model.opset)
        self.cuda = True
        self.do_auto_optimize = auto_optimize
        self.simplify = simplify
        self.save_transients = save_transients
        self.sdfg = sd.SDFG(name)  #: the generated SDFG
        self.sdfg._parent_onnx_model = self
        self.state = self.sdfg.add_state()  #: the state containing the model computation
        self.value_infos = dict(model.value_infos)
        self.inputs: List[str] = [v.name for v in model.inputs]  #: the inputs to the model
        self.outputs: List[str] = []  #: the outputs of the model (``__return*`` after import)
        self.weights: Dict[str, torch.Tensor] = {}  #: mapping from weight name to tensor
        self._compiled = None
        self._optimized = False

        # outputs are written straight into ``__return*`` (the reference copies them there in a second state)
        rename = {}
        for i, out in enumerate(model.outputs):
            new = "__return" if len(model.outputs) == 1 else "__return_{}".format(i)
            if out.name in rename or out.name in model.initializers or out.name in self.inputs:
                raise NotImplementedError("output '{}' is an input, a weight or listed twice".format(out.name))
            rename[out.name] = new
            self.outputs.append(new)
        self._rename = rename

        for v in model.inputs:
            self._add_value(v.name)
        for name, tensor in model.initializers.items():
            self._add_constant(name, tensor)

        access = {}

        def access_node(array):
            if array not in access:
                access[array] = self.state.add_access(array)
            return access[array]

        self._idx_to_node = []
        for i, node in enumerate(model.nodes):
            if node.op_type == "Constant":  # constants go to the weights immediately
                self._add_constant(node.outputs[0], _constant_value(node))
                continue
            if not has_onnx_node(node.op_type):
                raise ValueError("Unsupported ONNX operator: '{}'".format(node.op_type))
            cls = get_onnx_node(node.op_type)
            op_node = cls(clean_onnx_name(node.name) if node.name else "{}_{}".format(node.op_type, i), **node.attributes)
            self.state.add_node(op_node)
            self._idx_to_node.append(op_node)
            for is_input, names, params in ((True, node.inputs, cls.schema.inputs), (False, node.outputs, cls.schema.outputs)):
                for idx, vname in enumerate(names):
                    if vname is None:
                        continue
                    array = self._add_value(vname)
                    conn = self._connector(params, idx, is_input)
                    if is_input:
                        op_node.add_in_connector(conn)
                        self.state.add_edge(access_node(array), None, op_node, conn, self.sdfg.make_array_memlet(array))
                    else:
                        op_node.add_out_connector(conn)
                        self.state.add_edge(op_node, conn, access_node(array), None, self.sdfg.make_array_memlet(array))
        for out in self.outputs:
            if out not in self.sdfg.arrays:
                raise ValueError("model output '{}' is not produced by any node".format(out))
        self.sdfg.arg_names = [clean_onnx_name(i) for i in self.inputs]

    # -- construction helpers -------------------------------------------------------------------
    @staticmethod
    def _connector(params, idx, is_input):
        if idx >= len(params):
            if not params or params[-1].kind != VARIADIC:
                raise ValueError("Expected the last {io} parameter to be variadic, since the {io} with idx {i} has more "
                                 "parameters than the schema ({n})".format(io="input" if is_input else "output", i=idx,
                                                                            n=len(params)))
            return "{}__{}".format(params[-1].name, idx - len(params) + 1)
        if params[idx].kind == VARIADIC:
            return params[idx].name + "__0"
        return params[idx].name

    def _array_name(self, value_name):
        return self._rename.get(value_name) or clean_onnx_name(value_name)

    def _add_value(self, value_name):
        array = self._array_name(value_name)
        if array in self.sdfg.arrays:
            return array
        info = self.value_infos.get(value_name)
        if info is None:
            raise ValueError("Could not find array with name '{}'".format(value_name))
        if info.shape is None or info.dtype is None:
            raise ValueError("value '{}' has no static shape or type; export with fixed input shapes".format(value_name))
        transient = value_name not in self.inputs and value_name not in self._rename
        self.sdfg.add_array(array, tuple(info.shape), info.dtype, transient=transient)
        return array

    def _add_constant(self, value_name, tensor):
        if not isinstance(tensor, torch.Tensor):
            raise TypeError("weight '{}' is not a tensor".format(value_name))
        self.weights[value_name] = tensor
        self.sdfg.add_constant(clean_onnx_name(value_name), tensor.detach().contiguous())

    # -- the reference's public surface -----------------------------------------------------------
    @property
    def clean_weights(self):
        return {clean_onnx_name(k): v for k, v in self.weights.items()}

    def auto_optimize(self):
        from daceml_b200.util.utils import auto_optimize
        auto_optimize(self.sdfg, cuda=True, simplify=self.simplify)
        self._optimized = True

    def compile_and_init(self):
        """Compiles the SDFG (expanding what is still a library node); weights move to the device on first use."""
        if self._compiled is None:
            self._compiled = self.sdfg.compile()
        return self._compiled

    def __call__(self, *args, **kwargs):
        """Executes the model: the i-th positional argument is the i-th model input, keyword arguments go by ONNX
        name.  Returns the output, or a tuple of outputs."""
        if len(args) > len(self.inputs):
            raise ValueError("Expected {} arguments, got {}".format(len(self.inputs), len(args)))
        inputs = dict(kwargs)
        inputs.update(dict(zip(self.inputs, args)))
        missing = set(self.inputs) - set(inputs)
        if missing:
            raise ValueError("Missing inputs {}".format(", ".join(sorted(missing))))
        unknown = set(inputs) - set(self.inputs)
        if unknown:
            raise ValueError("Unknown inputs {}".format(", ".join(sorted(unknown))))
        if self.do_auto_optimize and not self._optimized:
            self.auto_optimize()
        compiled = self.compile_and_init()
        result = compiled(**{clean_onnx_name(k): v for k, v in inputs.items()})
        if self.save_transients is not None:
            self.save_transients.update(compiled._transients)
        return result

    # -- convenience ------------------------------------------------------------------------------
    @classmethod
    def from_torch(cls, name, module, dummy_inputs, **kwargs):
        """Exports ``module`` on ``dummy_inputs`` (opset 12, eval mode) and imports the result."""
        return cls(name, export_module(module, dummy_inputs), **kwargs)
