"""daceml_b200: a B200 (sm_100a) implementation of DaCeML's ONNX operator library-node forward path.

``import daceml_b200.onnx as donnx`` gives the node frontend; the kernels live in
``libdaceml_b200.so`` (``daceml_b200/csrc``) behind the C ABI of ``include/daceml_b200.h``.
There is no CPU or eager fallback: without the built library and a B200 every call raises.
"""
__version__ = "0.1.0"

import logging as _logging
import os as _os

# the reference's switch (daceml/__init__.py:9-11): DACEML_LOG_LEVEL=debug|info|... configures the root logger
if "DACEML_LOG_LEVEL" in _os.environ:
    _logging.basicConfig(level=getattr(_logging, _os.environ["DACEML_LOG_LEVEL"].upper(), _logging.INFO))
