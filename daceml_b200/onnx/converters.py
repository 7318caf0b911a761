"""Name and type conversions between exported graphs and SDFG arrays (``daceml/onnx/converters.py``)."""
import re

import torch


def clean_onnx_name(name: str) -> str:
    """Turns an ONNX value name into a valid array name, by the reference's rule
    (``daceml/onnx/converters.py:204-211``): a leading digit gets an ``ONNX_`` prefix and
    ``. : / -`` are spelled out."""
    if re.match("^[0-9]", name):
        name = "ONNX_" + name
    return name.replace(".", "DOT").replace(":", "COLON").replace("/", "SLASH").replace("-", "DASH")


# onnx.TensorProto.DataType values (the numbering is part of the ONNX file format)
ONNX_ELEM_TYPES = {
    1: torch.float32, 2: torch.uint8, 3: torch.int8, 5: torch.int16, 6: torch.int32, 7: torch.int64, 9: torch.bool,
    10: torch.float16, 11: torch.float64, 16: torch.bfloat16,
}


def onnx_tensor_type_to_torch(elem_type: int) -> torch.dtype:
    if elem_type not in ONNX_ELEM_TYPES:
        raise NotImplementedError("ONNX tensor element type {} is not supported".format(elem_type))
    return ONNX_ELEM_TYPES[elem_type]
