"""``import daceml_b200.onnx as donnx`` -- the ONNX library-node frontend.

Same surface as ``daceml.onnx`` (``daceml/onnx/__init__.py:1-9``): the ``ONNX<Op>`` node classes,
the implementation registry, and ``default_implementation``.  The reference's default is
``"pure"``; here it is ``"b200"``, the only implementation this package ships.
"""
from .nodes.onnx_op import *  # noqa: F401,F403
from .nodes.onnx_op import ONNXOp, has_onnx_node, get_onnx_node, program, Program  # noqa: F401
from .forward_implementation_abc import ONNXForward  # noqa: F401
from .op_implementations.utils import op_implementation  # noqa: F401
from .schema import SCHEMAS, ONNXSchema  # noqa: F401

default_implementation = "b200"

from . import op_implementations  # noqa: E402,F401  (registers the "b200" implementations)
