"""B200 implementations of the data-movement operators: Slice, Split, Concat, Expand, Gather, Where, MaxPool, Shape.

The reference writes these as memlet sub-range copies and mapped tasklets
(``daceml/onnx/op_implementations/pure_implementations.py:96-98, 260-281, 659-735, 781-1014``,
``img_op_implementations.py:28-161``).  Here each output is produced by one launch of a strided-copy,
gather, select or pooling kernel; sub-ranges and broadcasts are expressed as torch views (offset +
strides) of the caller's tensors, which is all the kernels need.  Where the reference restricts an
operator (Slice to axis 0 / step 1, Expand to the no-op case, MaxPool to no padding) the
implementation here takes the general ONNX form.
"""
import torch

from daceml_b200 import kernels as K, lib as L
from daceml_b200.onnx.forward_implementation_abc import ONNXForward
from daceml_b200.onnx.op_implementations.utils import op_implementation
from daceml_b200.sdfg import KernelTasklet
from daceml_b200.util.utils import in_desc_with_name, out_desc_with_name

_SIZES = (1, 2, 4, 8)
INT64_MAX = (1 << 63) - 1


def _movable(*descs):
    dt = descs[0].dtype
    return all(d.dtype == dt for d in descs) and torch.empty((), dtype=dt).element_size() in _SIZES and all(
        len(d.shape) <= 6 for d in descs)


def _const_input(node, state, sdfg, conn):
    for e in state.in_edges_by_connector(node, conn):
        return sdfg.constants.get(e.data.data)
    return None


def _has_input(node, state, conn):
    return any(True for _ in state.in_edges_by_connector(node, conn))


def _variadic(edges, conn_of):
    return [conn_of(e) for e in sorted(edges, key=lambda e: int(conn_of(e).split("__")[1]))]


# ---------------------------------------------------------------------------------------------
# Slice (pure_implementations.py:659-735 and 830-904)
# ---------------------------------------------------------------------------------------------
def slice_index(shape, starts, ends, axes=None, steps=None):
    """The tuple of Python slices ONNX Slice-10 describes (clamped starts / ends, ``INT64_MAX`` meaning "to the end");
    None when a step is not positive."""
    axes = list(range(len(starts))) if axes is None else [int(a) % len(shape) for a in axes]
    steps = [1] * len(starts) if steps is None else [int(s) for s in steps]
    index = [slice(None)] * len(shape)
    for s, e, a, st in zip(starts, ends, axes, steps):
        if st <= 0:
            return None
        n = shape[a]
        s, e = int(s), int(e)
        s = max(0, min(n, s + n if s < 0 else s))
        e = max(0, min(n, e + n if e < 0 else e))
        index[a] = slice(s, max(s, e), st)
    return tuple(index)


def _slice_plan(node, state, sdfg):
    data, out = in_desc_with_name(node, state, sdfg, "data"), out_desc_with_name(node, state, sdfg, "output")
    starts, ends = _const_input(node, state, sdfg, "starts"), _const_input(node, state, sdfg, "ends")
    if starts is None or ends is None:
        return None
    axes = steps = None
    if _has_input(node, state, "axes"):
        axes = _const_input(node, state, sdfg, "axes")
        if axes is None:
            return None
        axes = axes.tolist()
    if _has_input(node, state, "steps"):
        steps = _const_input(node, state, sdfg, "steps")
        if steps is None:
            return None
        steps = steps.tolist()
    index = slice_index(data.shape, starts.tolist(), ends.tolist(), axes, steps)
    if index is None:
        return None
    got = tuple(len(range(*sl.indices(n))) for sl, n in zip(index, data.shape))
    return index if got == tuple(out.shape) else None


@op_implementation(op="Slice", name="b200")
class B200Slice(ONNXForward):
    """Slice with constant ``starts / ends / axes / steps`` (any axes, positive steps) as one strided copy."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        return (_movable(in_desc_with_name(node, state, sdfg, "data"), out_desc_with_name(node, state, sdfg, "output"))
                and _slice_plan(node, state, sdfg) is not None)

    @staticmethod
    def forward(node, state, sdfg):
        index = _slice_plan(node, state, sdfg)

        def run(ins, outs):
            K.strided_copy(ins["data"][index], outs["output"])

        return KernelTasklet(node.label, run, kernels=("strided_copy", ))


# ---------------------------------------------------------------------------------------------
# Split / Concat (pure_implementations.py:781-827)
# ---------------------------------------------------------------------------------------------
def _split_sizes(node, state, sdfg):
    x = in_desc_with_name(node, state, sdfg, "input")
    conns = _variadic(state.out_edges(node), lambda e: e.src_conn)
    axis = int(node.axis) % len(x.shape)
    sizes = list(node.split) if node.split else None
    if sizes is None:
        if x.shape[axis] % len(conns):
            return None
        sizes = [x.shape[axis] // len(conns)] * len(conns)
    if len(sizes) != len(conns) or sum(sizes) != x.shape[axis]:
        return None
    for c, n in zip(conns, sizes):
        want = list(x.shape)
        want[axis] = n
        if tuple(out_desc_with_name(node, state, sdfg, c).shape) != tuple(want):
            return None
    return axis, conns, sizes


@op_implementation(op="Split", name="b200")
class B200Split(ONNXForward):
    """Split along ``axis`` into the sizes of the ``split`` attribute (equal parts when absent): one launch copies all parts."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x = in_desc_with_name(node, state, sdfg, "input")
        outs = [sdfg.arrays[e.data.data] for e in state.out_edges(node)]
        return bool(outs) and _movable(x, *outs) and _split_sizes(node, state, sdfg) is not None

    @staticmethod
    def forward(node, state, sdfg):
        axis, conns, sizes = _split_sizes(node, state, sdfg)

        def run(ins, outs):
            off, srcs, dsts = 0, [], []
            for c, n in zip(conns, sizes):
                srcs.append(ins["input"].narrow(axis, off, n))
                dsts.append(outs[c])
                off += n
            K.strided_copy_parts(srcs, dsts)  # every part in one launch (eight parts per launch)

        return KernelTasklet(node.label, run, kernels=("strided_copy", ) * ((len(conns) + 7) // 8))


def _concat_plan(node, state, sdfg):
    out = out_desc_with_name(node, state, sdfg, "concat_result")
    conns = _variadic(state.in_edges(node), lambda e: e.dst_conn)
    if node.axis is None or not conns:
        return None
    axis = int(node.axis) % len(out.shape)
    total = 0
    for c in conns:
        d = in_desc_with_name(node, state, sdfg, c)
        if len(d.shape) != len(out.shape) or any(a != b for i, (a, b) in enumerate(zip(d.shape, out.shape)) if i != axis):
            return None
        total += d.shape[axis]
    return (axis, conns) if total == out.shape[axis] else None


@op_implementation(op="Concat", name="b200")
class B200Concat(ONNXForward):
    """Concat along ``axis``: each input is copied into its sub-range of the output."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        ins = [sdfg.arrays[e.data.data] for e in state.in_edges(node)]
        return bool(ins) and _movable(out_desc_with_name(node, state, sdfg, "concat_result"), *ins) and _concat_plan(
            node, state, sdfg) is not None

    @staticmethod
    def forward(node, state, sdfg):
        axis, conns = _concat_plan(node, state, sdfg)

        def run(ins, outs):
            off, srcs, dsts = 0, [], []
            for c in conns:
                n = ins[c].shape[axis]
                srcs.append(ins[c])
                dsts.append(outs["concat_result"].narrow(axis, off, n))
                off += n
            K.strided_copy_parts(srcs, dsts)  # every part in one launch (eight parts per launch)

        return KernelTasklet(node.label, run, kernels=("strided_copy", ) * ((len(conns) + 7) // 8))


# ---------------------------------------------------------------------------------------------
# Expand (pure_implementations.py:260-281), Where (:96-98)
# ---------------------------------------------------------------------------------------------
@op_implementation(op="Expand", name="b200")
class B200Expand(ONNXForward):
    """Expand as a copy whose source strides are 0 on the broadcast axes (the ``shape`` input only fixes the output
    descriptor, which the importer already holds)."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x, y = in_desc_with_name(node, state, sdfg, "input"), out_desc_with_name(node, state, sdfg, "output")
        if not _movable(x, y):
            return False
        try:
            return tuple(torch.broadcast_shapes(tuple(x.shape), tuple(y.shape))) == tuple(y.shape)
        except RuntimeError:
            return False

    @staticmethod
    def forward(node, state, sdfg):
        def run(ins, outs):
            K.strided_copy(ins["input"].expand(outs["output"].shape), outs["output"])

        return KernelTasklet(node.label, run, kernels=("strided_copy", ))


@op_implementation(op="Where", name="b200")
class B200Where(ONNXForward):
    """``output = condition ? X : Y`` with numpy broadcasting."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        c, x, y, o = (in_desc_with_name(node, state, sdfg, "condition"), in_desc_with_name(node, state, sdfg, "X"),
                      in_desc_with_name(node, state, sdfg, "Y"), out_desc_with_name(node, state, sdfg, "output"))
        if c.dtype not in (torch.bool, torch.uint8) or not _movable(x, y, o) or torch.empty((), dtype=o.dtype).element_size() == 1:
            return False
        try:
            return tuple(torch.broadcast_shapes(tuple(c.shape), tuple(x.shape), tuple(y.shape))) == tuple(o.shape)
        except RuntimeError:
            return False

    @staticmethod
    def forward(node, state, sdfg):
        def run(ins, outs):
            K.where(ins["condition"], ins["X"], ins["Y"], outs["output"])

        return KernelTasklet(node.label, run, kernels=("where", ))


def _register_compare(op, code):
    def can(node, state, sdfg):
        a, b, c = (in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B"),
                   out_desc_with_name(node, state, sdfg, "C"))
        if a.dtype != b.dtype or a.dtype not in (torch.float16, torch.float32, torch.int64) or c.dtype != torch.bool:
            return False
        try:
            return len(c.shape) <= 6 and tuple(torch.broadcast_shapes(tuple(a.shape), tuple(b.shape))) == tuple(c.shape)
        except RuntimeError:
            return False

    def fwd(node, state, sdfg):
        def run(ins, outs):
            K.compare(ins["A"], ins["B"], outs["C"], code)

        return KernelTasklet(node.label, run, kernels=("compare", ))

    cls = type("B200" + op, (ONNXForward, ), dict(forward_can_be_applied=staticmethod(can), forward=staticmethod(fwd),
                                                 __doc__="Numpy-broadcast {} into a bool tensor (the condition of a Where); "
                                                 "the reference has no pure expansion for it.".format(op)))
    return op_implementation(op=op, name="b200")(cls)


B200Equal = _register_compare("Equal", L.CMP_EQ)
B200Greater = _register_compare("Greater", L.CMP_GT)
B200Less = _register_compare("Less", L.CMP_LT)
B200GreaterOrEqual = _register_compare("GreaterOrEqual", L.CMP_GE)
B200LessOrEqual = _register_compare("LessOrEqual", L.CMP_LE)


# ---------------------------------------------------------------------------------------------
# Gather (pure_implementations.py:949-1014), Shape (:907-946)
# ---------------------------------------------------------------------------------------------
@op_implementation(op="Gather", name="b200")
class B200Gather(ONNXForward):
    """``numpy.take(data, indices, axis)``; indices are int64 of any shape (scalar included)."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        d, i, o = (in_desc_with_name(node, state, sdfg, "data"), in_desc_with_name(node, state, sdfg, "indices"),
                   out_desc_with_name(node, state, sdfg, "output"))
        if i.dtype != torch.int64 or not _movable(d, o) or len(d.shape) == 0:
            return False
        axis = int(node.axis) % len(d.shape)
        return tuple(o.shape) == tuple(d.shape[:axis]) + tuple(i.shape) + tuple(d.shape[axis + 1:])

    @staticmethod
    def forward(node, state, sdfg):
        axis = int(node.axis)

        def run(ins, outs):
            K.gather(ins["data"], ins["indices"], outs["output"], axis)

        return KernelTasklet(node.label, run, kernels=("gather", ))


@op_implementation(op="Shape", name="b200")
class B200Shape(ONNXForward):
    """The (static) shape of ``data`` written as an int64 vector; normally folded away before expansion."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        o = out_desc_with_name(node, state, sdfg, "shape")
        return o.dtype == torch.int64 and tuple(o.shape) == (len(in_desc_with_name(node, state, sdfg, "data").shape), )

    @staticmethod
    def forward(node, state, sdfg):
        shape = list(in_desc_with_name(node, state, sdfg, "data").shape)
        cache = {}

        def run(ins, outs):
            dev = outs["shape"].device
            if dev not in cache:
                cache[dev] = torch.tensor(shape, dtype=torch.int64, device=dev)
            K.strided_copy(cache[dev], outs["shape"])

        return KernelTasklet(node.label, run, kernels=("strided_copy", ))


# ---------------------------------------------------------------------------------------------
# MaxPool (img_op_implementations.py:28-161)
# ---------------------------------------------------------------------------------------------
def _pool_geometry(node, x):
    kernel = [int(k) for k in (node.kernel_shape or [])]
    strides = [int(s) for s in (node.strides or [1, 1])]
    pads = [int(p) for p in (node.pads or [0, 0, 0, 0])]
    return kernel, strides, pads


@op_implementation(op="MaxPool", name="b200")
class B200MaxPool(ONNXForward):
    """2-D max pooling, floor mode, with ONNX padding (pads smaller than the kernel); no ``Indices`` output."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x, y = in_desc_with_name(node, state, sdfg, "X"), out_desc_with_name(node, state, sdfg, "Y")
        if any(e.src_conn == "Indices" for e in state.out_edges(node)):
            return False
        if x.dtype not in (torch.float16, torch.float32) or y.dtype != x.dtype or len(x.shape) != 4:
            return False
        if node.auto_pad != "NOTSET" or int(node.ceil_mode) != 0 or int(node.storage_order) != 0:
            return False
        if node.dilations is not None and any(int(d) != 1 for d in node.dilations):
            return False
        kernel, strides, pads = _pool_geometry(node, x)
        if len(kernel) != 2 or len(strides) != 2 or len(pads) != 4:
            return False
        if pads[0] >= kernel[0] or pads[2] >= kernel[0] or pads[1] >= kernel[1] or pads[3] >= kernel[1]:
            return False
        oh = (x.shape[2] + pads[0] + pads[2] - kernel[0]) // strides[0] + 1
        ow = (x.shape[3] + pads[1] + pads[3] - kernel[1]) // strides[1] + 1
        return tuple(y.shape) == (x.shape[0], x.shape[1], oh, ow)

    @staticmethod
    def forward(node, state, sdfg):
        kernel, strides, pads = _pool_geometry(node, in_desc_with_name(node, state, sdfg, "X"))

        def run(ins, outs):
            K.maxpool2d(ins["X"], outs["Y"], kernel=kernel, strides=strides, pads=pads)

        return KernelTasklet(node.label, run, kernels=("maxpool2d", ))
