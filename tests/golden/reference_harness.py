"""Runs the reference's own pure expansions under numpy, without DaCe and without the ``onnx`` package.

The arithmetic of the reference's pure expansions (``daceml/onnx/op_implementations/pure_implementations.py``,
``img_op_implementations.py``) is written as numpy-style Python that DaCe parses into an SDFG, or as code that
assembles a small nested SDFG (an Einsum node plus mapped tasklets).  Neither needs DaCe's code generator to be
*understood*: this module

* puts stand-ins for ``dace`` and the ``daceml`` modules those two files import into ``sys.modules``
  (data descriptors with ``shape`` / ``dtype``, a typeclass that converts a value, ``dace.elementwise``, a recording
  ``SDFG`` / ``SDFGState``, ``subsets.Range``, ``Memlet``),
* imports the two reference source files, unchanged and read-only, from a DaCeML checkout,
* replaces ``python_pure_op_implementation`` / ``program_for_node``
  (``daceml/onnx/op_implementations/utils.py:43-225``) by versions that keep the Python function and its
  ``compute`` lambdas, and executes the function body with numpy arrays,
* evaluates what the class-based expansions record (``PureMatMul``, ``PureGemm``, ``PureEinsum``, ``EinsumTranspose``,
  ``PureSum``, ``PureCast``, ``PureGather``, ``SplitPure``, ``PureSliceAllConstant``, ``PureShape``): the Einsum node's
  equation string with ``np.einsum``, every mapped tasklet point by point with its own code string, copies between
  ``Range`` subsets as slices,
* rewrites the explicit-dataflow syntax of ``PureConv2D`` (``for ... in dace.map[...]``, ``with dace.tasklet``,
  ``a << X[...]``, ``out >> Y(1, lambda x, y: x + y)[...]``) into plain Python loops that run sequentially, which is
  the order the write-conflict resolution of a sequential map gives.

Three adaptations are made, each where numpy and DaCe's numpy front end differ: a list given as ``axis`` becomes a
tuple; ``out[:] = value`` writes ``value`` into the output descriptor's own shape when only unit dimensions differ
(DaCe assigns into the descriptor, whose shape already carries ``keepdims``); and the C math functions named inside
``dace.elementwise`` lambdas (``sqrt``, ``exp``, ``erf``, ``tanh``, ``max``, ``min``) are bound to functions that keep
the element type.

This is test infrastructure: it is used by ``generate_from_reference.py`` only, to write fixtures.
"""
import ast
import importlib.util
import inspect
import itertools
import math
import os
import sys
import textwrap
import types

import numpy as np


# ------------------------------------------------------------------------------------------------
# dace stand-ins
# ------------------------------------------------------------------------------------------------
class TypeClass:
    """Stands in for ``dace.typeclass``: converts a value, names itself, indexes into an annotation."""

    def __init__(self, np_type):
        self.type = np_type

    def to_string(self):
        return np.dtype(self.type).name

    def __call__(self, value):
        return self.type(value)

    def __getitem__(self, shape):  # dace.float32[2, 3] as an annotation
        return ("annotation", self, shape)

    def __eq__(self, other):
        return isinstance(other, TypeClass) and np.dtype(other.type) == np.dtype(self.type)

    def __hash__(self):
        return hash(np.dtype(self.type))

    def __str__(self):
        return self.to_string()

    __repr__ = __str__


class Desc:
    """Stands in for ``dace.data.Array``."""

    def __init__(self, shape, dtype, transient=False):
        self.shape, self.dtype, self.transient = tuple(int(s) for s in shape), TypeClass(np.dtype(dtype).type), transient


class ScalarDesc(Desc):
    """Stands in for ``dace.data.Scalar``; its shape is (1,) as in DaCe."""

    def __init__(self, dtype):
        super().__init__((1,), dtype)


class Memlet:
    def __init__(self, expr=None, data=None, subset=None, other_subset=None, wcr=None):
        self.expr, self.data, self.subset, self.other_subset, self.wcr = expr, data, subset, other_subset, wcr
        if expr is not None and data is None:
            self.data = expr.split("[")[0].strip()

    def text(self):
        if self.expr is not None:
            return self.expr
        if self.subset is None:
            return self.data
        return "%s[%s]" % (self.data, self.subset)


class Range:
    """``dace.subsets.Range``: inclusive (begin, end, step) triples."""

    def __init__(self, ranges):
        self.ranges = [tuple(int(v) for v in r) for r in ranges]

    @staticmethod
    def from_array(desc):
        return Range([(0, s - 1, 1) for s in desc.shape])

    def slices(self):
        return tuple(slice(b, e + 1, s) for b, e, s in self.ranges)


class AccessNode:
    def __init__(self, data):
        self.data = data


class EinsumNode:
    """What ``onnx_op.ONNXEinsum(label, equation=...)`` leaves behind."""

    def __init__(self, label, equation=None):
        self.label, self.equation = label, equation

    def add_in_connector(self, name):
        pass


class Tasklet:
    def __init__(self, name, inputs, outputs, code, map_ranges=None):
        self.name, self.inputs, self.outputs, self.code, self.map_ranges = name, inputs, outputs, code, map_ranges
        self.in_connectors, self.out_connectors = {}, {}


class RecState:
    """Records what an expansion builds, in creation order."""

    def __init__(self, sdfg):
        self.sdfg, self.ops, self.edges, self.access = sdfg, [], [], []

    def add_node(self, node):
        self.ops.append(node)

    def _access(self, name):
        node = AccessNode(name)
        self.access.append(node)
        return node

    add_read = add_write = add_access = _access

    def add_edge(self, src, src_conn, dst, dst_conn, memlet):
        self.edges.append((src, src_conn, dst, dst_conn, memlet))

    def add_nedge(self, src, dst, memlet):
        self.ops.append(("copy", src, dst, memlet))
        self.edges.append((src, None, dst, None, memlet))

    def add_mapped_tasklet(self, name, map_ranges, inputs, code, outputs, external_edges=False, input_nodes=None, **kw):
        ranges = list(map_ranges.items()) if isinstance(map_ranges, dict) else list(map_ranges)
        t = Tasklet(name, dict(inputs), dict(outputs), code, ranges)
        self.ops.append(t)
        for m in t.inputs.values():
            src = None
            for cand in (input_nodes or {}).values():
                if cand.data == m.data:
                    src = cand
            self.edges.append((src or self._access(m.data), None, t, None, m))
        for m in t.outputs.values():
            self.edges.append((t, None, self._access(m.data), None, m))
        return t, None, None

    def add_tasklet(self, name, inputs, outputs, code, **kw):
        t = Tasklet(name, dict.fromkeys(inputs), dict.fromkeys(outputs), code)
        self.ops.append(t)
        return t

    def sink_nodes(self):
        with_out = {id(e[0]) for e in self.edges}
        return [n for n in self.access if id(n) not in with_out]


class RecSDFG:
    def __init__(self, name="sdfg"):
        self.name, self.arrays, self.state_list = name, {}, []

    def add_state(self, *a, **k):
        s = RecState(self)
        self.state_list.append(s)
        return s

    def add_datadesc(self, name, desc):
        self.arrays[name] = desc
        return name

    def add_array(self, name, shape, dtype, transient=False, **k):
        self.arrays[name] = Desc(shape, dtype.type if isinstance(dtype, TypeClass) else dtype, transient)
        return name, self.arrays[name]

    def make_array_memlet(self, name):
        return Memlet(data=name)


class SchedulingOnly(Exception):
    """Raised when an expansion starts to transform the SDFG of an already captured program (map expansion and
    collapsing in ``PureConv2D.forward``): those steps change the schedule, not the result."""


class CapturedProgram:
    """What ``program_for_node(program, sdfg, state, node, extra_vars)`` returns here."""

    def __init__(self, fn, extra_vars):
        self.fn, self.extra_vars = fn, dict(extra_vars or {})

    def __getattr__(self, name):
        raise SchedulingOnly(name)


def _keep_type(fn):
    def wrapped(x, *rest):
        return type(x)(fn(float(x), *rest)) if isinstance(x, np.generic) else fn(x, *rest)
    return wrapped


class NumpyProxy:
    """numpy, with a list accepted wherever DaCe's numpy front end accepts one as ``axis``."""

    class _Ufunc:
        def __init__(self, uf):
            self.uf = uf

        def __call__(self, *a, **k):
            return self.uf(*a, **k)

        def reduce(self, x, axis=0, **k):
            return self.uf.reduce(x, axis=_tuple_axis(axis), **k)

    def __getattr__(self, name):
        obj = getattr(np, name)
        if name in ("mean", "sum", "max", "min"):
            return lambda x, axis=None, **k: obj(x, axis=_tuple_axis(axis), **k)
        if name in ("maximum", "add"):
            return NumpyProxy._Ufunc(obj)
        if name == "transpose":
            return lambda x, axes=None: obj(x, axes=None if axes is None else tuple(axes))
        if name == "reshape":
            return lambda x, shape: obj(np.asarray(x), tuple(int(s) for s in shape))
        return obj


def _tuple_axis(axis):
    return tuple(axis) if isinstance(axis, list) else axis


class Output:
    """The array behind an output connector.  ``out[:] = value`` stores into the descriptor's shape."""

    def __init__(self, shape, dtype):
        self.array = np.zeros(shape, dtype=dtype)
        self.shape, self.dtype = self.array.shape, self.array.dtype

    def __setitem__(self, key, value):
        value = np.asarray(value)
        whole = isinstance(key, slice) and key == slice(None)
        if whole and value.shape != self.array.shape and value.size == self.array.size:
            drop = lambda s: tuple(d for d in s if d != 1)
            assert drop(value.shape) == drop(self.array.shape), (value.shape, self.array.shape)
            value = value.reshape(self.array.shape)
        self.array[key] = value

    def __getitem__(self, key):
        return self.array[key]


# ------------------------------------------------------------------------------------------------
# the explicit-dataflow syntax as plain Python
# ------------------------------------------------------------------------------------------------
class _Dataflow(ast.NodeTransformer):
    def visit_FunctionDef(self, node):
        node.decorator_list = []
        for a in node.args.args:
            a.annotation = None
        node.returns = None
        self.generic_visit(node)
        return node

    def visit_For(self, node):
        self.generic_visit(node)
        it = node.iter
        if (isinstance(it, ast.Subscript) and isinstance(it.value, ast.Attribute) and it.value.attr == "map"
                and isinstance(it.value.value, ast.Name) and it.value.value.id == "dace"):
            dims = it.slice.elts if isinstance(it.slice, ast.Tuple) else [it.slice]
            names = node.target.elts if isinstance(node.target, ast.Tuple) else [node.target]
            body = node.body
            for name, dim in reversed(list(zip(names, dims))):
                rng = ast.Call(func=ast.Name(id="range", ctx=ast.Load()), args=[dim.lower, dim.upper], keywords=[])
                body = [ast.For(target=name, iter=rng, body=body, orelse=[])]
            return body[0]
        return node

    def visit_With(self, node):
        ctx = node.items[0].context_expr
        if not (isinstance(ctx, ast.Attribute) and ctx.attr == "tasklet"):
            return self.generic_visit(node)
        body, writes = [], []
        for stmt in node.body:
            if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.BinOp) and isinstance(stmt.value.op, ast.LShift):
                body.append(ast.Assign(targets=[ast.Name(id=stmt.value.left.id, ctx=ast.Store())], value=stmt.value.right))
            elif isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.BinOp) and isinstance(stmt.value.op, ast.RShift):
                writes.append((stmt.value.left.id, stmt.value.right))
            else:
                body.append(stmt)
        for name, target in writes:
            value = ast.Name(id=name, ctx=ast.Load())
            if isinstance(target.value, ast.Call):  # Y(1, lambda x, y: x + y)[idx]: write-conflict resolution
                array, wcr = target.value.func, target.value.args[1]
                old = ast.Subscript(value=array, slice=target.slice, ctx=ast.Load())
                value = ast.Call(func=wcr, args=[old, value], keywords=[])
                target = ast.Subscript(value=array, slice=target.slice, ctx=ast.Store())
            else:
                target = ast.Subscript(value=target.value, slice=target.slice, ctx=ast.Store())
            body.append(ast.Assign(targets=[target], value=value))
        return ast.If(test=ast.Constant(value=True), body=body, orelse=[])


def as_python(fn, extra=None):
    """The function ``fn`` (plain numpy-style Python or explicit dataflow) as an executable Python function whose
    globals are the reference module's, the enclosing function's variables, and ``extra``."""
    if isinstance(fn, DaceProgram):
        fn = fn.fn
    tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    tree = ast.fix_missing_locations(_Dataflow().visit(tree))
    env = dict(fn.__globals__)
    if fn.__closure__:
        for name, cell in zip(fn.__code__.co_freevars, fn.__closure__):
            try:
                env[name] = cell.cell_contents
            except ValueError:
                pass
    env.update(GLOBALS)
    env.update(extra or {})
    exec(compile(tree, inspect.getsourcefile(fn) or "<reference>", "exec"), env)
    return env[fn.__name__]


class DaceProgram:
    """``@dace.program`` here: a function that runs through ``as_python`` when called."""

    def __init__(self, fn):
        self.fn = fn

    def __call__(self, *args):
        return as_python(self.fn)(*args)


def elementwise(func, x):
    """``dace.elementwise(func, X)``: ``func`` (a lambda or the source of one) on every element, in X's type."""
    if isinstance(func, str):
        func = eval(func, dict(GLOBALS))
    x = np.asarray(x)
    out = np.empty_like(x)
    flat_in, flat_out = x.reshape(-1), out.reshape(-1)
    for i in range(flat_in.size):
        flat_out[i] = func(flat_in[i])
    return out


DACE = types.ModuleType("dace")
GLOBALS = {}


def _build_dace():
    d = DACE
    for name in ("float16", "float32", "float64", "int8", "int16", "int32", "int64", "uint8", "bool_"):
        setattr(d, name, TypeClass(getattr(np, name)))
    d.bool = d.bool_
    d.elementwise, d.Memlet, d.SDFG, d.SDFGState, d.program = elementwise, Memlet, RecSDFG, RecState, DaceProgram
    d.DeviceType = types.SimpleNamespace(CPU="CPU")
    mods = {}

    def sub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        mods[name] = m
        parent, _, leaf = name.rpartition(".")
        setattr(mods[parent] if parent in mods else d, leaf, m)
        return m

    mods["dace"] = d
    nodes = sub("dace.nodes", AccessNode=AccessNode, Node=object, LibraryNode=object, EntryNode=type("EntryNode", (), {}))
    sub("dace.subsets", Range=Range)
    sub("dace.data", Scalar=ScalarDesc, Array=Desc)
    sub("dace.symbolic", issymbolic=lambda v: False)
    sub("dace.dtypes", paramdec=None, ScheduleType=types.SimpleNamespace(GPU_Default="gpu"), GPU_SCHEDULES=[],
        min_value=lambda t: np.finfo(t.type).min if np.issubdtype(t.type, np.floating) else np.iinfo(t.type).min)
    sub("dace.registry", autoregister=lambda cls, **k: cls)
    sub("dace.frontend")
    sub("dace.frontend.common", create_einsum_sdfg=_create_einsum_sdfg)
    sd = sub("dace.sdfg", nodes=nodes)
    mods["dace.sdfg.nodes"] = nodes
    sub("dace.sdfg.propagation")
    sub("dace.transformation")
    sub("dace.transformation.dataflow", MapExpansion=object, MapCollapse=object)
    sd.SDFG, sd.SDFGState = RecSDFG, RecState
    GLOBALS.update(dace=d, np=NumpyProxy(), sqrt=np.sqrt, exp=np.exp, log=np.log, tanh=np.tanh,
                   erf=_keep_type(math.erf), max=max, min=min)
    return mods


def _create_einsum_sdfg(_, sdfg, state, equation, *inputs, output="Output"):
    state.ops.append(("einsum", equation, list(inputs), output))


# ------------------------------------------------------------------------------------------------
# daceml stand-ins: only what the two source files import
# ------------------------------------------------------------------------------------------------
REGISTRY = {}


class PurePython:
    """What ``@python_pure_op_implementation`` keeps: the function and its ``compute`` lambdas."""

    def __init__(self, func, compute):
        self.func, self.compute = func, compute


def _op_implementation(op, name):
    def dec(cls):
        REGISTRY.setdefault((op, name), []).append(cls)
        return cls
    return dec


def _python_pure_op_implementation(func=None, **compute):
    if func is None:
        return lambda f: _python_pure_op_implementation(f, **compute)
    impl = PurePython(func, compute)
    REGISTRY.setdefault((func.__name__, "pure"), []).append(impl)
    return impl


def _program_for_node(program, sdfg, state, node, extra_vars=None):
    return CapturedProgram(program, extra_vars)


def _empty_sdfg_for_node(sdfg, state, node, add_access_nodes=True):
    nsdfg = RecSDFG(node.label + "_expansion")
    nstate = nsdfg.add_state()
    for name, d in list(node.in_descs.items()) + list(node.out_descs.items()):
        nsdfg.add_datadesc(name, d)
    return nsdfg, nstate, {}, {}


def _in_desc(node, state, sdfg, name):
    if name not in node.in_descs:
        raise ValueError("no edge to connector " + name)
    return node.in_descs[name]


def _out_desc(node, state, sdfg, name):
    if name not in node.out_descs:
        raise ValueError("no edge from connector " + name)
    return node.out_descs[name]


class Edge:
    def __init__(self, src, src_conn, dst, dst_conn):
        self.src, self.src_conn, self.dst, self.dst_conn = src, src_conn, dst, dst_conn
        self.data = types.SimpleNamespace(data=src.data if isinstance(src, AccessNode) else dst.data)


def _in_edge_with_name(node, state, name):
    if name not in node.in_descs:
        raise ValueError("no edge to connector " + name)
    return Edge(AccessNode(name), None, node, name)


class Node:
    """An ONNX library node with its edges: descriptors by connector name, attributes as properties."""

    def __init__(self, op, inputs, outputs, constants=None, **attrs):
        self.op, self.label, self.name = op, op.lower() + "_node", op.lower() + "_node"
        self.inputs = {k: np.asarray(v) for k, v in inputs.items()}
        self.in_descs = {k: (ScalarDesc(v.dtype) if v.ndim == 0 else Desc(v.shape, v.dtype)) for k, v in self.inputs.items()}
        self.out_descs = {k: Desc(shape, dtype) for k, (shape, dtype) in outputs.items()}
        self.in_connectors, self.out_connectors = dict.fromkeys(self.in_descs), dict.fromkeys(self.out_descs)
        self.constants = set(constants or ())
        self.schedule = None
        self.__dict__.update(attrs)

    def iter_inputs_in_onnx_order(self, state):
        return [Edge(AccessNode(k), None, self, k) for k in self.in_descs]

    def iter_outputs_in_onnx_order(self, state):
        return [Edge(self, k, AccessNode(k), None) for k in self.out_descs]


class State:
    """The state around the node: enough for expansions that look at their neighbours."""

    def __init__(self, node):
        self.node = node

    def node_id(self, node):
        return 0

    def in_edges_by_connector(self, node, conn):
        return iter([Edge(AccessNode(conn), None, node, conn)] if conn in node.in_descs else [])

    def out_edges(self, node):
        return node.iter_outputs_in_onnx_order(self)

    def predecessors(self, n):
        return []


def _onnx_constant_or_none(sdfg, access):
    node = sdfg.node
    if access.data not in node.constants:
        return None
    v = node.inputs[access.data]
    return v.item() if v.size == 1 else list(v.tolist())


def _prod(seq):
    out = 1
    for s in seq:
        out *= s
    return out


def install(reference_root):
    """Puts the stand-ins into ``sys.modules`` and imports the two reference source files.  Returns them."""
    mods = _build_dace()
    DACE.dtypes.paramdec = lambda f: f
    for name, m in mods.items():
        sys.modules[name] = m

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []
        sys.modules[name] = m
        return m

    onnx_op = module("daceml.onnx.nodes.onnx_op", ONNXOp=Node, ONNXEinsum=EinsumNode)
    module("daceml")
    module("daceml.onnx", converters=None)
    module("daceml.onnx.converters", onnx_tensor_type_to_typeclass=lambda t: t)
    sys.modules["daceml.onnx"].converters = sys.modules["daceml.onnx.converters"]
    module("daceml.onnx.nodes", onnx_op=onnx_op)
    module("daceml.onnx.forward_implementation_abc", ONNXForward=object)
    module("daceml.onnx.op_implementations")
    module("daceml.onnx.op_implementations.utils", op_implementation=_op_implementation, program_for_node=_program_for_node,
           empty_sdfg_for_node=_empty_sdfg_for_node, python_pure_op_implementation=_python_pure_op_implementation)
    cf = module("daceml.transformation.constant_folding", remove_node_and_computation=lambda *a, **k: None)
    module("daceml.transformation", constant_folding=cf)
    module("daceml.transformation.replacement", onnx_constant_or_none=_onnx_constant_or_none)
    module("daceml.util")
    module("daceml.util.utils", in_desc_with_name=_in_desc, out_desc_with_name=_out_desc, in_edge_with_name=_in_edge_with_name,
           out_edge_with_name=None, iterables_equal=lambda a, b: list(a) == list(b), prod=_prod)
    loaded = []
    for leaf in ("pure_implementations", "img_op_implementations"):
        path = os.path.join(reference_root, "daceml", "onnx", "op_implementations", leaf + ".py")
        spec = importlib.util.spec_from_file_location("daceml.onnx.op_implementations." + leaf, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        loaded.append(mod)
    return loaded


# ------------------------------------------------------------------------------------------------
# evaluation
# ------------------------------------------------------------------------------------------------
def _call(fn, node, extra):
    py = as_python(fn, extra)
    outs = {k: Output(d.shape, d.dtype.type) for k, d in node.out_descs.items()}
    args = []
    for name in inspect.signature(fn).parameters:
        args.append(node.inputs[name] if name in node.inputs else outs[name])
    py(*args)
    return {k: v.array for k, v in outs.items()}


def _eval_recorded(nsdfg, node):
    arrays = dict(node.inputs)
    for name, d in nsdfg.arrays.items():
        if name not in arrays:
            arrays[name] = np.zeros(d.shape, dtype=d.dtype.type)
    scalars = {k for k, d in node.in_descs.items() if isinstance(d, ScalarDesc)}
    for k in scalars:  # a DaCe scalar is indexed as [0]
        arrays[k] = np.asarray(arrays[k]).reshape(1)
    for state in nsdfg.state_list:
        for op in state.ops:
            if isinstance(op, EinsumNode):
                ins = sorted((e for e in state.edges if e[2] is op), key=lambda e: e[3])
                out = next(e for e in state.edges if e[0] is op)
                operands = [arrays[e[0].data] for e in ins]
                arrays[out[2].data][...] = np.einsum(op.equation, *operands)
            elif isinstance(op, tuple) and op[0] == "einsum":
                _, equation, ins, out = op
                arrays[out][...] = np.einsum(equation, *[arrays[i] for i in ins])
            elif isinstance(op, tuple) and op[0] == "copy":
                _, src, dst, m = op
                arrays[dst.data][m.other_subset.slices()] = arrays[src.data][m.subset.slices()]
            elif isinstance(op, Tasklet) and op.map_ranges is not None:
                names = [n for n, _ in op.map_ranges]
                extents = [range(*[int(v) for v in r.split(":")]) for _, r in op.map_ranges]
                for point in itertools.product(*extents):
                    env = dict(arrays)
                    env.update(zip(names, point))
                    local = {"dace": DACE}
                    for conn, m in op.inputs.items():
                        local[conn] = eval(m.text(), {}, env)
                    exec(op.code, dict(GLOBALS), local)
                    for conn, m in op.outputs.items():
                        env["__value"] = local[conn]
                        exec("%s = __value" % m.text(), {}, env)
            elif isinstance(op, Tasklet):  # a tasklet without a map: its output memlet hangs on an edge
                local = {}
                exec(op.code, dict(GLOBALS), local)
                for e in state.edges:
                    if e[0] is op:
                        env = dict(arrays)
                        env["__value"] = local[e[1]]
                        exec("%s = __value" % e[4].text(), {}, env)
            else:
                raise NotImplementedError(op)
    return {k: arrays[k] for k in node.out_descs}


def run(op, inputs, outputs, implementation="pure", constants=None, **attrs):
    """Runs the reference expansion ``implementation`` of ONNX operator ``op``.

    ``inputs``: connector name -> array; ``outputs``: connector name -> (shape, dtype); ``constants``: names of inputs
    that are constants of the model (Clip's bounds, Slice's parameters); ``attrs``: the node's ONNX attributes.
    Returns connector name -> array.  Raises ``LookupError`` if no registered implementation applies."""
    node = Node(op, inputs, outputs, constants=constants, **attrs)
    state, sdfg = State(node), types.SimpleNamespace(node=node)
    for impl in REGISTRY.get((op, implementation), []):
        if isinstance(impl, PurePython):
            extra = {}
            for var, fn in impl.compute.items():
                args = []
                for a in inspect.signature(fn).parameters:
                    args.append(node if a == "node" else node.in_descs[a] if a in node.in_descs else node.out_descs[a])
                extra[var] = fn(*args)
            return _call(impl.func, node, extra)
        can = getattr(impl, "forward_can_be_applied", None)
        if can is not None and not can(node, state, sdfg):
            continue
        captured = []
        original = sys.modules["daceml.onnx.op_implementations.utils"].program_for_node
        module_globals = impl.forward.__globals__

        def capture(program, sdfg_, state_, node_, extra_vars=None):
            captured.append(CapturedProgram(program, extra_vars))
            return captured[-1]

        module_globals["program_for_node"] = capture
        try:
            result = impl.forward(node, state, sdfg)
        except SchedulingOnly:
            result = captured[-1]
        finally:
            module_globals["program_for_node"] = original
        if isinstance(result, CapturedProgram):
            return _call(result.fn, node, result.extra_vars)
        return _eval_recorded(result, node)
    raise LookupError("no applicable '%s' implementation of %s" % (implementation, op))
