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
