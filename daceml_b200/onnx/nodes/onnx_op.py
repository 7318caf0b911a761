"""ONNX library nodes: one ``ONNX<Op>`` class per schema, with the reference's selection rules.

Mirrors ``daceml/onnx/nodes/onnx_op.py``:

* a node is built as ``donnx.ONNXConv("label", strides=[2, 2])`` and wired with
  ``state.add_edge(access, None, node, "X", memlet)`` (``onnx_op.py:434-491`` shows the connector
  names being taken from the schema);
* ``node.expand(sdfg, state)`` validates the node, asks the selected implementation whether it
  can be applied and calls its ``forward`` (the wrapper at ``onnx_op.py:668-697``).  The
  reference falls back to ONNX Runtime when ``forward_can_be_applied`` is false; this build has
  no fallback and raises instead;
* the implementation is chosen per instance (``node.implementation``), per class
  (``ONNXConv.default_implementation``) or library-wide (``donnx.default_implementation``).

Calling a node class with tensors, ``donnx.ONNXConv(X=x, W=w, Y=y, strides=[2, 2])``, is the
counterpart of the python-frontend replacement (``onnx_op.py:434-491``): outside a traced program
it builds a one-node SDFG, expands it and runs it on the tensors' device.
"""
import itertools
import logging

import numpy as np
import torch

from daceml_b200 import sdfg as sd
from daceml_b200.onnx.schema import SCHEMAS, OPTIONAL, VARIADIC, ONNXSchema

log = logging.getLogger(__name__)

_ONNX_OPS_BY_NAME = {}


def parse_variadic_param(param):
    """``"Inputs__3"`` -> ``("Inputs", 3)`` (``daceml/onnx/nodes/node_utils.py``)."""
    split = param.split("__")
    if len(split) != 2:
        raise ValueError("Unable to parse variadic parameter '{}'".format(param))
    return split[0], int(split[1])


class Expansion:
    """Base of the per-(op, implementation) expansion classes, like ``ExpandTransformation``."""
    environments = []
    forward_impl = None

    @classmethod
    def expansion(cls, node, state, sdfg, **kwargs):
        node.validate(sdfg, state)
        if cls.forward_impl.forward_can_be_applied(node, state, sdfg):
            return cls.forward_impl.forward(node, state, sdfg, **kwargs)
        raise NotImplementedError(
            'Library node "{}": implementation "{}" cannot be applied (forward_can_be_applied returned False) '
            'and this build has no ONNX Runtime fallback'.format(node.label, cls.__name__))


class _ONNXOpMeta(type):
    """Makes ``ONNXConv(X=tensor, ...)`` run the operator, while ``ONNXConv("label", ...)`` builds a node."""

    def __call__(cls, *args, **kwargs):
        if cls.schema is not None and not args and any(_is_array(v) for v in kwargs.values()):
            return _frontend_call(cls, kwargs)
        return super().__call__(*args, **kwargs)


def _is_array(v):
    return isinstance(v, (torch.Tensor, np.ndarray, TracedArray))


class ONNXOp(sd.Node, metaclass=_ONNXOpMeta):
    """ Abstract superclass for all ONNX ops."""
    schema: ONNXSchema = None
    implementations = {}
    default_implementation = None

    def __init__(self, name, *args, location=None, **op_attributes):
        self.label = name
        self.name = name
        self.implementation = None
        self.location = location or {}
        self.in_connectors = {}
        self.out_connectors = {}
        unknown = set(op_attributes) - set(self.schema.attributes)
        if unknown:
            raise TypeError("{} got unknown attribute(s) {}".format(type(self).__name__, sorted(unknown)))
        for attr, default in self.schema.attributes.items():
            val = op_attributes.get(attr, default)
            if isinstance(val, tuple):
                val = list(val)
            setattr(self, attr, val)

    def __repr__(self):
        return "{}({})".format(type(self).__name__, self.label)

    # -- connectors ----------------------------------------------------------------------------
    def add_in_connector(self, name):
        self.in_connectors[name] = None
        return True

    def add_out_connector(self, name):
        self.out_connectors[name] = None
        return True

    def iter_edges(self, state, ignore_unknown=False):
        """Yields ``(edge, is_input)`` for every edge of this node."""
        for e in state.in_edges(self):
            yield e, True
        for e in state.out_edges(self):
            yield e, False

    def _ordered(self, edges, params, conn_of):
        order = {p.name: i for i, p in enumerate(params)}

        def key(e):
            conn = conn_of(e)
            if "__" in conn:
                base, idx = parse_variadic_param(conn)
                return order.get(base, 1 << 20), idx
            return order.get(conn, 1 << 20), 0

        return sorted(edges, key=key)

    def iter_inputs_in_onnx_order(self, state):
        return self._ordered(state.in_edges(self), self.schema.inputs, lambda e: e.dst_conn)

    def iter_outputs_in_onnx_order(self, state):
        return self._ordered(state.out_edges(self), self.schema.outputs, lambda e: e.src_conn)

    # -- validation (onnx_op.py:213-431: connectors, then the schema's type constraints, then required attributes) ------
    def validate(self, sdfg, state):
        self._validate_connectors(sdfg, state)
        # type parameters: connectors that share one must agree, and the element type must be one it allows
        assigned = {}
        for edges, conn_of, what in ((state.in_edges(self), lambda e: e.dst_conn, "input"),
                                     (state.out_edges(self), lambda e: e.src_conn, "output")):
            for e in edges:
                conn = conn_of(e)
                base = parse_variadic_param(conn)[0] if "__" in conn else conn
                tparam = self.schema.type_params[base]
                dtype = sdfg.arrays[e.data.data].dtype
                if tparam in assigned and assigned[tparam] != dtype:
                    raise ValueError("Could not solve type constraints; expected type '{}' for {} '{}', got type '{}'".format(
                        assigned[tparam], what, base, dtype))
                possible = self.schema.type_constraints[tparam]
                if dtype not in possible:
                    raise ValueError("Expected type in '{}' for {} '{}', got type '{}'".format(
                        [str(t) for t in possible], what, base, dtype))
                assigned[tparam] = dtype
        for attr in self.schema.required_attributes:
            if getattr(self, attr, None) is None:
                raise ValueError("Expected value for required attribute '{}', got None".format(attr))

    def _validate_connectors(self, sdfg, state):
        for params, edges, conn_of, what in ((self.schema.inputs, state.in_edges(self), lambda e: e.dst_conn, "input"),
                                             (self.schema.outputs, state.out_edges(self), lambda e: e.src_conn,
                                              "output")):
            present = {}
            for e in edges:
                conn = conn_of(e)
                if conn is None:
                    raise ValueError("{}: {} edge without a connector".format(self, what))
                base = parse_variadic_param(conn)[0] if "__" in conn else conn
                present.setdefault(base, []).append(conn)
                if e.data.data not in sdfg.arrays:
                    raise ValueError("{}: memlet names unknown array '{}'".format(self, e.data.data))
            names = {p.name: p for p in params}
            for base in present:
                if base not in names:
                    raise ValueError("{}: unknown {} connector '{}'".format(self, what, base))
                if names[base].kind != VARIADIC and len(present[base]) > 1:
                    raise ValueError("{}: {} connector '{}' is connected more than once".format(self, what, base))
            for p in params:
                if p.kind not in (OPTIONAL, VARIADIC) and p.name not in present:
                    raise ValueError("{}: required {} connector '{}' is not connected".format(self, what, p.name))
                if p.kind == VARIADIC and p.name not in present:
                    raise ValueError("{}: variadic {} connector '{}' needs at least one edge".format(self, what, p.name))

    # -- implementation selection and expansion --------------------------------------------------
    @classmethod
    def register_implementation(cls, name, expansion_cls):
        if "implementations" not in cls.__dict__:
            cls.implementations = dict(cls.implementations)
        cls.implementations[name] = expansion_cls

    def selected_implementation(self):
        import daceml_b200.onnx as donnx
        return self.implementation or type(self).default_implementation or donnx.default_implementation

    def expand(self, sdfg, state, **kwargs):
        impl = self.selected_implementation()
        if impl not in type(self).implementations:
            raise KeyError('{} has no implementation "{}" (registered: {})'.format(
                type(self).__name__, impl, sorted(type(self).implementations)))
        result = type(self).implementations[impl].expansion(self, state, sdfg, **kwargs)
        if isinstance(result, sd.SDFG):
            result = _nested_sdfg_tasklet(self, result)
        if not isinstance(result, sd.KernelTasklet):
            raise TypeError("expansion of {} returned {}, expected a KernelTasklet".format(self, type(result)))
        state.replace_node(self, result)
        return impl


def _nested_sdfg_tasklet(node, nsdfg):
    """An expansion may return an SDFG whose non-transient arrays are named after the node's connectors (see
    ``empty_sdfg_for_node``); it is compiled here (its own library nodes expand, its transients are allocated) and runs in
    the node's place."""
    compiled = nsdfg.compile()

    def run(ins, outs):
        args = dict(ins)
        args.update(outs)
        compiled(**{k: v for k, v in args.items() if k in nsdfg.arrays})

    return sd.KernelTasklet(node.label + "_expansion", run, kernels=tuple(compiled.kernel_names()))


def attach_implementation(op, name, forward_cls):
    """Creates the ``Expansion`` of a registered implementation and attaches it to ``ONNX<op>``."""
    cls = _ONNX_OPS_BY_NAME.get("ONNX" + op)
    if cls is None:
        return False
    exp = type("Expansion_{}_{}".format(op, name), (Expansion,), dict(forward_impl=forward_cls, environments=[]))
    cls.register_implementation(name, exp)
    return True


def has_onnx_node(name: str) -> bool:
    """ Check if an ONNX operator is supported. """
    return ("ONNX" + name) in _ONNX_OPS_BY_NAME


def get_onnx_node(name: str):
    """ Get the ONNX Operator node for an operator by name. """
    return _ONNX_OPS_BY_NAME["ONNX" + name]


# ------------------------------------------------------------------------------------------------
# Class generation: one ONNX<Op> per schema (onnx_op.py:510-711)
# ------------------------------------------------------------------------------------------------
for _schema in SCHEMAS.values():
    _cls_name = "ONNX" + _schema.name
    _cls = _ONNXOpMeta(_cls_name, (ONNXOp, ), dict(schema=_schema, implementations={}, default_implementation=None,
                                                  __doc__="ONNX operator {}.".format(_schema.name)))
    globals()[_cls_name] = _cls
    _ONNX_OPS_BY_NAME[_cls_name] = _cls

# implementations registered before this module finished importing
from daceml_b200.onnx.forward_implementation_abc import ONNXForward  # noqa: E402

for _impl, _args in list(ONNXForward.extensions().items()):
    if "op" in _args:
        attach_implementation(_args["op"], _args["name"], _impl)


# ------------------------------------------------------------------------------------------------
# Frontend: eager call and tracing
# ------------------------------------------------------------------------------------------------
class TracedArray:
    """Placeholder for an array while a :func:`program` is traced into an SDFG."""

    def __init__(self, builder, name, shape, dtype):
        self.builder, self.name, self.shape, self.dtype = builder, name, tuple(shape), sd.to_torch_dtype(dtype)


class _Builder:
    active = None

    def __init__(self, name):
        self.sdfg = sd.SDFG(name)
        self.state = self.sdfg.add_state()
        self.counter = itertools.count()


def _split_kwargs(cls, kwargs):
    schema = cls.schema
    attrs = {k: v for k, v in kwargs.items() if k in schema.attributes}
    in_names = {p.name for p in schema.inputs}
    out_names = {p.name for p in schema.outputs}
    inputs, outputs = {}, {}
    for k, v in kwargs.items():
        if k in attrs:
            continue
        base = parse_variadic_param(k)[0] if "__" in k else k
        if base in in_names:
            inputs[k] = v
        elif base in out_names:
            outputs[k] = v
        else:
            raise TypeError("{}: '{}' is neither a connector nor an attribute".format(cls.__name__, k))
    return attrs, inputs, outputs


def _frontend_call(cls, kwargs):
    attrs, inputs, outputs = _split_kwargs(cls, kwargs)
    traced = [v for v in itertools.chain(inputs.values(), outputs.values()) if isinstance(v, TracedArray)]
    if traced:
        b = traced[0].builder
        node = cls("{}_{}".format(cls.schema.name, next(b.counter)), **attrs)
        b.state.add_node(node)
        for conn, arr in inputs.items():
            b.state.add_edge(b.state.add_read(arr.name), None, node, conn, b.sdfg.make_array_memlet(arr.name))
        for conn, arr in outputs.items():
            b.state.add_edge(node, conn, b.state.add_write(arr.name), None, b.sdfg.make_array_memlet(arr.name))
        return None
    # eager: a one-node SDFG over the given tensors
    g = sd.SDFG("eager_" + cls.schema.name)
    st = g.add_state()
    node = cls(cls.schema.name, **attrs)
    st.add_node(node)
    call_args = {}
    for conn, val in itertools.chain(inputs.items(), outputs.items()):
        name = "arr_" + conn
        host = isinstance(val, np.ndarray) or not val.is_cuda
        if conn in inputs and host and not torch.as_tensor(val).is_floating_point():
            # index-like operands held on the host (Slice starts / ends, Reshape and Expand shapes, Gather indices) are
            # values known when the node is built: constants, as an importer would bind them
            g.add_constant(name, torch.as_tensor(val))
        else:
            g.add_array(name, val.shape, val.dtype)
            call_args[name] = val
        if conn in inputs:
            st.add_edge(st.add_read(name), None, node, conn, g.make_array_memlet(name))
        else:
            st.add_edge(node, conn, st.add_write(name), None, g.make_array_memlet(name))
    g.compile()(**call_args)
    return None


class Program:
    """Counterpart of ``@dace.program`` for functions made of ``donnx.ONNX*`` calls.

    The argument annotations give shapes and types as ``(dtype, shape)`` pairs;
    ``to_sdfg()`` traces the function once into an SDFG of library nodes."""

    def __init__(self, fn):
        self.fn = fn
        self.name = fn.__name__
        self._compiled = None

    def to_sdfg(self):
        b = _Builder(self.name)
        args = {}
        for pname, ann in self.fn.__annotations__.items():
            dtype, shape = ann
            b.sdfg.add_array(pname, shape, dtype)
            args[pname] = TracedArray(b, pname, shape, dtype)
        self.fn(**args)
        return b.sdfg

    def __call__(self, **kwargs):
        if self._compiled is None:
            self._compiled = self.to_sdfg().compile()
        return self._compiled(**kwargs)


def program(fn):
    return Program(fn)
