"""``DaceModule``: wraps an ``nn.Module`` so that its forward pass runs on this library's kernels.

Mirror of the reference's class of the same name (``daceml/torch/module.py:46-365``): the wrapped
module is exported to ONNX operators at opset 12 on the first call (or on ``dummy_inputs``), the
graph is imported as an SDFG of ONNX library nodes (:class:`daceml_b200.onnx.ONNXModel`),
``post_onnx_hooks`` run (``auto_optimize`` is the default hook), the SDFG is compiled and
``post_compile_hooks`` run.  Later calls only launch kernels.

Differences, all consequences of this being the forward operator path only: ``backward=True`` and
``training=True`` raise (there is no autodiff and no training-mode BatchNorm / Dropout kernel);
parameters are bound as constants when the SDFG is built, so call :meth:`reset_sdfg` after changing
the wrapped module's weights; ``cuda_graph=True`` (an addition) replays the launches as one CUDA
graph over static input and output buffers.
"""
import collections
import functools
import logging
from typing import Callable, List, Optional, Tuple

import torch
import torch.nn as nn

from daceml_b200.onnx.exported_graph import export_module
from daceml_b200.onnx.onnx_importer import ONNXModel
from daceml_b200.util import utils

log = logging.getLogger(__name__)


def _find_str_not_in_set(existing, target):
    """``target``, or ``target_<i>`` with the first free i (``daceml/util/utils.py`` ``find_str_not_in_set``)."""
    if target not in existing:
        return target
    i = 0
    while "{}_{}".format(target, i) in existing:
        i += 1
    return "{}_{}".format(target, i)


class DaceModule(nn.Module):
    """A wrapper that converts a PyTorch ``nn.Module`` to a PyTorch compatible module running on B200 kernels.

    :param module: the model to wrap.
    :param dummy_inputs: a tuple of tensors to use as input when tracing ``model``.
    :param cuda: must be ``True`` or ``None``; the wrapped module is moved to the current CUDA device.
    :param training: must be ``False``.
    :param backward: must be ``False``.
    :param auto_optimize: whether to apply automatic optimizations (constant folding, fusion, expansion).
    :param debug_transients: if True, the module will have all transients as outputs.
    :param sdfg_name: the name to give to the sdfg (defaults to the module's class name).
    :param cuda_graph: replay the forward pass as one CUDA graph (inputs are copied into static buffers and the
                       returned tensors are reused by the next call).
    :param compile_torch_extension: call the compiled module through a registered torch operator
                                    (``torch.ops.daceml_<sdfg_name>.<sdfg_name>``), as the reference's C++ extension does.
    ``inputs_to_skip``, ``onnx_simplify`` and ``simplify`` are accepted for signature compatibility.

    :Example:

        >>> from daceml_b200.torch import DaceModule
        >>> dace_module = DaceModule(module.cuda())
        >>> dace_module(torch.ones(2, device="cuda"))
    """

    def __init__(self, module: nn.Module, dummy_inputs: Optional[Tuple[torch.Tensor, ...]] = None, cuda: Optional[bool] = None,
                 training: bool = False, backward=False, inputs_to_skip: Optional[List[str]] = None, onnx_simplify: bool = True,
                 simplify: bool = True, auto_optimize: bool = True, debug_transients: bool = False,
                 compile_torch_extension: bool = True, sdfg_name: Optional[str] = None, cuda_graph: bool = False):
        super().__init__()
        if backward:
            raise NotImplementedError("daceml_b200 implements the forward operator path; backward=True needs autodiff")
        if training:
            raise NotImplementedError("daceml_b200 imports inference graphs only (training=False)")
        if cuda is not None and not cuda:
            raise ValueError("daceml_b200 has no CPU path: DaceModule needs cuda=True")
        self.backward = False
        self.model = module
        self.dace_model: Optional[ONNXModel] = None
        self.training = False
        self.sdfg = None
        self.use_cuda = True
        self.sdfg_name = sdfg_name or type(module).__name__
        self.auto_optimize = auto_optimize
        self.onnx_simplify = onnx_simplify
        self.simplify = simplify
        self.debug_transients = debug_transients
        self.compile_torch_extension = compile_torch_extension
        self.inputs_to_skip = inputs_to_skip or []
        self.cuda_graph = cuda_graph
        self.function = None
        self.compiled_function = None

        #: hooks that are executed after onnx graph is imported to an SDFG
        self.post_onnx_hooks: "collections.OrderedDict[str, Callable[[DaceModule], None]]" = collections.OrderedDict()
        #: hooks that are executed after the sdfg is compiled
        self.post_compile_hooks: "collections.OrderedDict[str, Callable]" = collections.OrderedDict()

        if self.debug_transients:

            def transients_outputs(module):
                for name, desc in module.sdfg.arrays.items():
                    if desc.transient and len(desc.shape) > 0:
                        desc.transient = False
                        module.dace_model.outputs.append(name)

            self.prepend_post_onnx_hook("make_transients_outputs", transients_outputs)

        if self.auto_optimize:
            self.append_post_onnx_hook(
                "auto_optimize", lambda dace_module: utils.auto_optimize(dace_module.dace_model.sdfg, True, simplify=self.simplify))

        if dummy_inputs is not None:
            self.function = self._initialize_sdfg(dummy_inputs)

    def train(self, mode: bool = True):
        if mode:
            raise NotImplementedError("daceml_b200 runs inference graphs only")
        return self

    def reset_sdfg(self):
        """ Clear the sdfg so that optimizations are reapplied (and the wrapped module's weights are read again). """
        self.function = None
        self._release_torch_op()

    def _release_torch_op(self):
        handle = getattr(self, "torch_op_handle", None)
        if handle is not None:
            from .dispatchers import release_torch_op
            release_torch_op(handle)
            self.torch_op = self.torch_op_handle = None

    def __del__(self):
        try:
            self._release_torch_op()
        except Exception:
            pass

    def check_status(self, synchronize=True):
        """Raises :class:`daceml_b200.lib.B200Error` if a kernel of this module's device recorded a problem since the
        last check: a Gather index outside its axis (the kernel wrote zeros there) or a device-side wait that gave up.
        Kernels report through a status word instead of stopping the process, so a caller that wants to know calls
        this after its work (``synchronize=False`` if the stream is already idle).  Clears the word."""
        compiled = getattr(self, "compiled_function", None)
        if compiled is None:
            return
        compiled.check_status(synchronize=synchronize)

    # -- hooks (``daceml/torch/module.py:179-235``) ------------------------------------------------
    def _add_hook(self, hooks, name, func, first):
        if self.function is not None:
            log.warning("Added a hook after the model was already initialized. This hook (with name %s) will not be "
                        "executed!", name)
        name = _find_str_not_in_set(set(hooks), name)
        hooks[name] = func
        if first:
            hooks.move_to_end(name, last=False)

    def prepend_post_onnx_hook(self, name: str, func: Callable[["DaceModule"], None]):
        self._add_hook(self.post_onnx_hooks, name, func, True)

    def append_post_onnx_hook(self, name: str, func: Callable[["DaceModule"], None]):
        self._add_hook(self.post_onnx_hooks, name, func, False)

    def prepend_post_compile_hook(self, name: str, func: Callable):
        self._add_hook(self.post_compile_hooks, name, func, True)

    def append_post_compile_hook(self, name: str, func: Callable):
        self._add_hook(self.post_compile_hooks, name, func, False)

    def prepend_post_autodiff_hook(self, name, func):
        raise NotImplementedError("there is no backward pass to hook into")

    append_post_autodiff_hook = prepend_post_autodiff_hook

    # -- building ------------------------------------------------------------------------------------
    def _initialize_sdfg(self, dummy_inputs):
        if not isinstance(dummy_inputs, (tuple, list)):
            dummy_inputs = (dummy_inputs, )
        if torch.cuda.is_available():
            self.model = self.model.cuda()
            dummy_inputs = tuple(t.cuda() if isinstance(t, torch.Tensor) else t for t in dummy_inputs)
        graph = export_module(self.model, tuple(dummy_inputs))
        dace_model = ONNXModel(self.sdfg_name, graph, cuda=True, auto_optimize=self.auto_optimize,
                               onnx_simplify=self.onnx_simplify)
        # the hooks below do the optimisation (``module.py:317-326``); the model itself must not repeat it per call
        dace_model.do_auto_optimize = False
        self.sdfg = dace_model.sdfg
        self.dace_model = dace_model
        for _, hook in self.post_onnx_hooks.items():
            hook(self)
        compiled = dace_model.compile_and_init()
        self.compiled_function = compiled
        for _, hook in self.post_compile_hooks.items():
            hook(compiled)

        input_names = list(self.sdfg.arg_names)
        output_names = list(dace_model.outputs)

        def run(*args):
            if len(args) != len(input_names):
                raise ValueError("Expected {} arguments, got {}".format(len(input_names), len(args)))
            kwargs = dict(zip(input_names, args))
            outs = {}
            if len(output_names) != 1 or output_names[0] != "__return" or self.debug_transients:
                dev = compiled._device()
                for name in output_names:
                    desc = self.sdfg.arrays[name]
                    outs[name] = torch.empty(desc.shape, dtype=desc.dtype, device=dev)
            result = compiled(**kwargs, **outs)
            if outs:
                vals = tuple(outs[n] for n in output_names)
                return vals[0] if len(vals) == 1 else vals
            return result

        if not self.cuda_graph:
            return self._as_torch_op(run, input_names, output_names)

        from daceml_b200.runner import GraphedCall
        dev = compiled._device()
        static_in = [torch.zeros(self.sdfg.arrays[n].shape, dtype=self.sdfg.arrays[n].dtype, device=dev) for n in input_names]
        for buf, t in zip(static_in, dummy_inputs):
            buf.copy_(t)
        holder = {}

        def step():
            holder["out"] = run(*static_in)

        graphed = GraphedCall(step)
        self._graphed = graphed

        def replay(*args):
            if len(args) != len(static_in):
                raise ValueError("Expected {} arguments, got {}".format(len(static_in), len(args)))
            for buf, t in zip(static_in, args):
                if t.data_ptr() != buf.data_ptr():
                    buf.copy_(t, non_blocking=True)
            graphed()
            return holder["out"]

        self.static_inputs = static_in
        return self._as_torch_op(replay, input_names, output_names)

    def _as_torch_op(self, function, input_names, output_names):
        """With ``compile_torch_extension`` (the default, as in the reference) the module is called through a registered
        torch operator, ``torch.ops.daceml_<sdfg_name>.<sdfg_name>(handle, *inputs)``; otherwise directly."""
        self.torch_op = None
        if not self.compile_torch_extension or self.debug_transients:
            return function
        from .dispatchers import register_torch_op
        outs = [(self.sdfg.arrays[n].shape, self.sdfg.arrays[n].dtype) for n in output_names]
        try:
            op, handle = register_torch_op(self.sdfg_name, input_names, outs, function)
        except Exception as e:  # an operator schema torch rejects must not make the module unusable
            log.warning("could not register %s as a torch operator (%s); calling it directly", self.sdfg_name, e)
            return function
        self.torch_op, self.torch_op_handle = op, handle

        def call(*args):
            if not all(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
                return function(*args)  # host tensors are staged by the compiled SDFG itself
            result = op(handle, *args)
            return tuple(result) if isinstance(result, list) else result

        return call

    def forward(self, *actual_inputs):
        """ Execute the forward pass using the traced ``module``."""
        if self.function is None:
            self.function = self._initialize_sdfg(actual_inputs)
        return self.function(*actual_inputs)


def dace_module(moduleclass=None, dummy_inputs: Optional[Tuple[torch.Tensor]] = None, cuda: Optional[bool] = None,
                training: bool = False, backward=False, inputs_to_skip: Optional[List[str]] = None, onnx_simplify: bool = True,
                simplify: bool = True, auto_optimize: bool = True, sdfg_name: Optional[str] = None,
                compile_torch_extension: bool = True, debug_transients: bool = False, cuda_graph: bool = False):
    """ Decorator to apply on a definition of a ``torch.nn.Module`` to convert it to a :class:`DaceModule` upon
        construction (``daceml/torch/module.py:508-567``); usable bare or with keyword arguments.

        :Example:

            >>> @dace_module
            ... class MyDecoratedModule(nn.Module):
            ...     def forward(self, x):
            ...        return torch.sqrt(torch.log(x))
    """
    def decorate(cls):
        @functools.wraps(cls)
        def _create(*args, **kwargs):
            return DaceModule(cls(*args, **kwargs), dummy_inputs=dummy_inputs, cuda=cuda, training=training, backward=backward,
                              inputs_to_skip=inputs_to_skip, onnx_simplify=onnx_simplify, simplify=simplify,
                              auto_optimize=auto_optimize, sdfg_name=sdfg_name, compile_torch_extension=compile_torch_extension,
                              debug_transients=debug_transients, cuda_graph=cuda_graph)

        return _create

    return decorate(moduleclass) if moduleclass is not None else decorate
