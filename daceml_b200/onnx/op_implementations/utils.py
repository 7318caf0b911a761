"""``@op_implementation`` -- the registration decorator of the reference
(``daceml/onnx/op_implementations/utils.py:19-40``), plus late attachment to the node class.

In the reference the loop that turns registry entries into expansions runs once, when
``onnx_op.py`` is imported (``daceml/onnx/nodes/onnx_op.py:664-701``), so an implementation
registered later is visible in ``ONNXForward.extensions()`` but not selectable on the node.  Here
the decorator also attaches the implementation to ``ONNX<op>`` when that class already exists.
"""
from daceml_b200.onnx.forward_implementation_abc import ONNXForward


def op_implementation(op, name):
    """ A decorator that registers an op implementation.
        It should be used on classes that extend :class:`ONNXForward`.

        :param op: the ONNX name of the op to register for.
        :param name: the name of the implementation.
    """
    def dec(cls):
        doc = "\n                :Implementation name: ``\"{}\"``\n                ".format(name)
        cls.__doc__ = (cls.__doc__ or "") + doc
        ONNXForward.register(cls, op=op, name=name)
        from daceml_b200.onnx.nodes import onnx_op
        onnx_op.attach_implementation(op, name, cls)
        return cls

    return dec


# ---------------------------------------------------------------------------------------------
# Helpers for writing an implementation in a few lines of Python
# (counterparts of ``daceml/onnx/op_implementations/utils.py:43-225``)
# ---------------------------------------------------------------------------------------------
def parse_variadic_param(param):
    """``"Inputs__2"`` -> ``("Inputs", 2)``: the name a variadic connector gets per operand."""
    split = param.split("__")
    if len(split) != 2:
        raise ValueError("Unable to parse variadic parameter '{}'".format(param))
    name = split[0]
    number = split[1]
    if number[0] == "0" and len(number) > 1:
        raise ValueError("Variadic parameters must not be numbered with leading zeroes, got: '{}'".format(number))
    return name, int(number)


def program_for_node(program, sdfg, state, node, extra_vars=None):
    """Turns a Python function into the expansion of ``node``.

    The reference parses ``program`` with DaCe's Python frontend into a nested SDFG
    (``utils.py:43-104``).  Here the function is what runs: its parameters are named after the node's connectors and
    receive the device tensors bound to them (inputs and, pre-allocated, outputs, which it fills in place: ``Y[:] = ...``
    or a call into :mod:`daceml_b200.kernels`).  Parameter names are checked against the schema as the reference does,
    with its messages; ``extra_vars`` become global names of the function.  Inputs the function does not name are
    simply not read.  Returns the :class:`~daceml_b200.sdfg.KernelTasklet` that takes the node's place."""
    import inspect
    import types
    from daceml_b200 import sdfg as sd

    input_names = node.schema.non_variadic_inputs()
    variadic_input_names = node.schema.variadic_inputs()
    output_names = node.schema.non_variadic_outputs()
    variadic_output_names = node.schema.variadic_outputs()
    both = set(input_names).intersection(output_names)
    if both:
        raise ValueError("program_for_node cannot be applied on nodes of this type;"
                         " '{}' are both an input and an output".format(both))
    params = list(inspect.signature(program).parameters)
    in_params, out_params = [], []
    for name in params:
        if name in input_names or ("__" in name and parse_variadic_param(name)[0] in variadic_input_names):
            in_params.append(name)
        elif name in output_names or ("__" in name and parse_variadic_param(name)[0] in variadic_output_names):
            out_params.append(name)
        else:
            raise ValueError("'{}' was not found as an input or output for {}".format(name, node.schema.name))
    fn = program
    if extra_vars:
        scope = dict(program.__globals__)
        scope.update(extra_vars)
        fn = types.FunctionType(program.__code__, scope, program.__name__, program.__defaults__, program.__closure__)
        fn.__kwdefaults__ = program.__kwdefaults__

    def run(ins, outs):
        args = {}
        for name in in_params:
            if name not in ins:
                raise KeyError("{}: input connector '{}' is not connected".format(node.label, name))
            args[name] = ins[name]
        for name in out_params:
            if name not in outs:
                raise KeyError("{}: output connector '{}' is not connected".format(node.label, name))
            args[name] = outs[name]
        fn(**args)

    return sd.KernelTasklet(node.label + "_expansion", run, kernels=(program.__name__, ))


def empty_sdfg_for_node(sdfg, state, node, add_access_nodes=True):
    """An SDFG to build the expansion of ``node`` in: one non-transient array per connected connector, named after
    it and described like the array on the other end of the edge, and (unless ``add_access_nodes`` is false) an access
    node for each.  Returns ``(nsdfg, nstate, input_nodes, output_nodes)`` like ``utils.py:107-139``.  An expansion may
    return the filled SDFG; it runs in the node's place with the connectors' tensors as arguments."""
    import copy
    from daceml_b200 import sdfg as sd
    from daceml_b200.util.utils import in_desc_with_name, out_desc_with_name

    nsdfg = sd.SDFG(node.label + "_expansion")
    nstate = nsdfg.add_state()
    input_nodes, output_nodes = {}, {}
    for edge, is_input in node.iter_edges(state, ignore_unknown=True):
        if is_input:
            conn = edge.dst_conn
            nsdfg.add_datadesc(conn, copy.deepcopy(in_desc_with_name(node, state, sdfg, conn)))
            if add_access_nodes:
                input_nodes[conn] = nstate.add_read(conn)
        else:
            conn = edge.src_conn
            nsdfg.add_datadesc(conn, copy.deepcopy(out_desc_with_name(node, state, sdfg, conn)))
            if add_access_nodes:
                output_nodes[conn] = nstate.add_write(conn)
        nsdfg.arrays[conn].transient = False
        nsdfg.arrays[conn].view_of = None
    return nsdfg, nstate, input_nodes, output_nodes


def python_pure_op_implementation(func=None, **compute):
    """Registers ``func`` as the ``"pure"`` implementation of the operator it is named after (``utils.py:142-225``).

    ``func`` takes the node's connectors by name (see :func:`program_for_node`).  Each ``compute`` entry is a function
    whose own parameters are ``node`` and / or connector names (it receives the node, or the connector's data
    descriptor); its value becomes a global name of ``func``::

        @python_pure_op_implementation(axis=lambda node: node.axis)
        def Softmax(input, output):
            output[:] = torch.softmax(input, axis)

    Use as ``@python_pure_op_implementation`` or with compute entries as above."""
    import inspect
    import textwrap
    from daceml_b200.util.utils import in_desc_with_name, out_desc_with_name

    def dec(f):
        @op_implementation(op=f.__name__, name="pure")
        class PureImpl(ONNXForward):
            @staticmethod
            def forward(node, state, sdfg):
                def resolve(arg):
                    if arg == "node":
                        return node
                    if arg in node.in_connectors:
                        return in_desc_with_name(node, state, sdfg, arg)
                    if arg in node.out_connectors:
                        return out_desc_with_name(node, state, sdfg, arg)
                    raise ValueError("Got unknown compute argument {}. Arguments to compute can be either 'node',"
                                     " or the name of a connector of the node".format(arg))

                extra_vars = {}
                for var_name, function in compute.items():
                    names = list(inspect.signature(function).parameters)
                    extra_vars[var_name] = function(*[resolve(n) for n in names])
                return program_for_node(f, sdfg, state, node, extra_vars=extra_vars)

        try:
            source = textwrap.indent(inspect.getsource(f), prefix="    ")
        except (OSError, TypeError):
            source = "    (source not available)"
        PureImpl.__module__ = f.__module__
        PureImpl.__name__ = f.__name__
        PureImpl.__qualname__ = f.__qualname__
        PureImpl.__doc__ = "\nPure implementation made with :func:`python_pure_op_implementation`.\n\n.. code :: python\n\n" + source
        return PureImpl

    if func is not None:
        if compute:
            raise TypeError("pass the function alone, or only compute entries")
        return dec(func)
    return dec
