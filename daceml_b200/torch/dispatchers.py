"""Registers a compiled module as a torch operator, ``torch.ops.daceml_<name>.<name>(handle_ptr, *inputs)``.

The reference generates and compiles a C++ extension per module whose ``TORCH_LIBRARY`` block declares exactly this
operator and whose implementation calls the compiled SDFG (``daceml/torch/dispatchers/cpp_torch_extension.py:398-457``,
the state handle passed as an integer, ``:425``).  The SDFG here is a launch plan in Python, so the operator is declared
with ``torch.library`` instead; the effect for the caller is the same: the module is one opaque operator with a schema
and a shape function, which is what ``torch.compile``, tracing and export need in order to keep it as a single call.
"""
import itertools
import logging
from typing import Callable, List, Sequence, Tuple

import torch

log = logging.getLogger(__name__)

_HANDLES = {}  # handle_ptr -> callable(*tensors)
_handle_ids = itertools.count(1)
_LIBRARIES = []  # keeps the torch.library.Library objects (and with them the registrations) alive
_used_namespaces = set()
_LIB_OF_HANDLE = {}


def _identifier(name: str) -> str:
    out = "".join(c if c.isalnum() or c == "_" else "_" for c in name)
    return out if out and not out[0].isdigit() else "m_" + out


def register_torch_op(sdfg_name: str, input_names: Sequence[str], outputs: List[Tuple[tuple, torch.dtype]],
                      function: Callable) -> Tuple[Callable, int]:
    """Declares ``daceml_<sdfg_name>::<sdfg_name>(int handle_ptr, Tensor <input>...) -> Tensor | Tensor[]`` with a CUDA
    implementation that calls ``function(*inputs)`` and a meta implementation that returns empty tensors of the
    ``outputs`` shapes and types.  Returns the operator and the handle to pass as its first argument.  A second module
    with the same SDFG name gets a numbered namespace (an operator cannot be declared twice)."""
    name = _identifier(sdfg_name)
    ns = "daceml_" + name
    for i in itertools.count():
        cand = ns if i == 0 else "{}_{}".format(ns, i)
        if cand not in _used_namespaces:
            ns = cand
            break
    _used_namespaces.add(ns)
    args = ", ".join("Tensor " + _identifier(a) for a in input_names)
    ret = "Tensor" if len(outputs) == 1 else "Tensor[]"
    lib = torch.library.Library(ns, "DEF")
    lib.define("{}(int handle_ptr{}) -> {}".format(name, (", " + args) if args else "", ret))
    handle = next(_handle_ids)
    _HANDLES[handle] = function

    def run(handle_ptr, *tensors):
        result = _HANDLES[handle_ptr](*tensors)
        if len(outputs) == 1:
            return result
        return list(result)

    def meta(handle_ptr, *tensors):
        made = [torch.empty(shape, dtype=dtype, device="meta") for shape, dtype in outputs]
        return made[0] if len(outputs) == 1 else made

    lib.impl(name, run, "CUDA")
    lib.impl(name, meta, "Meta")
    _LIBRARIES.append(lib)
    _LIB_OF_HANDLE[handle] = lib
    return getattr(getattr(torch.ops, ns), name), handle


def release_torch_op(handle: int) -> None:
    """Forgets the compiled function behind ``handle`` (and with it the weights and transients it keeps on the GPU)
    and drops the operator's registration.  Called when a module is reset or collected; the namespace is not reused."""
    _HANDLES.pop(handle, None)
    lib = _LIB_OF_HANDLE.pop(handle, None)
    if lib is not None:
        if lib in _LIBRARIES:
            _LIBRARIES.remove(lib)
        destroy = getattr(lib, "_destroy", None)
        if destroy is not None:
            try:
                destroy()
            except Exception as e:  # pragma: no cover - torch keeps the registration; only the memory matters here
                log.debug("could not drop operator library: %s", e)
