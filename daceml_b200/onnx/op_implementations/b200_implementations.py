"""The ``"b200"`` implementations of the ONNX library nodes.

Each class is registered with ``@op_implementation(op=..., name="b200")`` exactly as the
reference registers its ``"pure"`` and ``"cuDNN"`` implementations
(``daceml/onnx/op_implementations/pure_implementations.py``, ``img_op_implementations.py``,
``cudnn_implementations.py``).  ``forward`` reads shapes and types from the node's edges
(``in_desc_with_name`` / ``out_desc_with_name``), works out the launch parameters once, and returns
a :class:`~daceml_b200.sdfg.KernelTasklet` whose callable enqueues hand-written sm_100a kernels
through the C ABI.  ``forward_can_be_applied`` says no where the library has no kernel; nothing
falls back to another backend.
"""
import math

import torch

from daceml_b200 import kernels as K
from daceml_b200 import lib as L
from daceml_b200.onnx.forward_implementation_abc import ONNXForward
from daceml_b200.onnx.op_implementations.utils import op_implementation
from daceml_b200.sdfg import KernelTasklet
from daceml_b200.util.utils import in_desc_with_name, out_desc_with_name, prod

FLOAT_TYPES = (torch.float16, torch.float32)


def _has_in(node, state, conn):
    return any(True for _ in state.in_edges_by_connector(node, conn))


def _has_out(node, state, conn):
    return any(True for _ in state.out_edges_by_connector(node, conn))


def _float_descs(*descs):
    return all(d.dtype in FLOAT_TYPES for d in descs) and len({d.dtype for d in descs}) == 1


def _norm_axis(a, rank):
    return a + rank if a < 0 else a


# ---------------------------------------------------------------------------------------------
# MatMul / Gemm / Einsum (pure_implementations.py:111-252, 380-553)
# ---------------------------------------------------------------------------------------------
def _matmul_plan(a_shape, b_shape):
    """Maps a numpy-style matmul onto (batch_outer, m, k, n, a_batched, b_batched) or None."""
    if len(a_shape) < 2 or len(b_shape) < 2:
        return None  # the reference rejects 1-D operands as well (:116-121)
    m, k = a_shape[-2:]
    kb, n = b_shape[-2:]
    if k != kb:
        return None
    ab, bb = tuple(a_shape[:-2]), tuple(b_shape[:-2])
    if not bb:  # [..., M, K] @ [K, N]: one flat GEMM, as the 'zik,kj->zij' einsum specialises to
        return dict(batch=1, m=prod(ab) * m, k=k, n=n, a_batched=False, b_batched=False)
    if not ab:
        return dict(batch=prod(bb), m=m, k=k, n=n, a_batched=False, b_batched=True)
    if ab == bb:
        return dict(batch=prod(ab), m=m, k=k, n=n, a_batched=True, b_batched=True)
    return None


def _b_is_constant(node, state, sdfg, conn="B"):
    """Whether the array on ``conn`` is a constant of the SDFG (a weight bound at build time): no kernel of the graph
    writes it, so a GEMM may fetch it before the kernel in front of it has finished."""
    for e in state.in_edges_by_connector(node, conn):
        return e.data.data in sdfg.constants
    return False


def _launch_gemm(a, b, out, plan, *, b_layout=0, a_layout=0, alpha=1.0, bias=None, bias_scale=1.0, residual=None,
                 residual_scale=1.0, act=0, ln=None, b_constant=False):
    ctx = L.get_context(a.device)
    p = L.GemmParams()
    p.dtype = L.dtype_code(a.dtype)
    p.flags = L.GEMM_B_CONSTANT if b_constant else 0
    p.a_layout, p.b_layout = a_layout, b_layout
    m, k, n = plan["m"], plan["k"], plan["n"]
    p.m, p.n, p.k = m, n, k
    p.batch_outer, p.batch_inner = plan["batch"], 1
    p.lda = m if a_layout else k
    p.ldb = k if b_layout else n
    p.ldc = n
    p.a_stride_outer = m * k if plan["a_batched"] else 0
    p.b_stride_outer = k * n if plan["b_batched"] else 0
    p.c_stride_outer = m * n
    p.epilogue = act | (L.EPI_BIAS if bias is not None else 0) | (L.EPI_RESIDUAL if residual is not None else 0)
    p.alpha, p.bias_scale, p.residual_scale = alpha, bias_scale, residual_scale
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    if residual is not None:
        p.residual, p.ldr, p.r_stride_outer = residual.data_ptr(), n, m * n
    if ln is not None:  # (gamma, beta, eps): LayerNorm over the finished row inside the GEMM epilogue
        p.epilogue |= L.EPI_LAYERNORM
        p.ln_gamma = ln[0].data_ptr() if ln[0] is not None else None
        p.ln_beta = ln[1].data_ptr() if ln[1] is not None else None
        p.ln_eps = ln[2]
    K.gemm_raw(ctx, p, L.current_stream(a.device))


@op_implementation(op="MatMul", name="b200")
class B200MatMul(ONNXForward):
    """MatMul on tcgen05 tensor cores (fp16) or FP32 FMA (fp32); B is consumed in its ONNX [K, N] layout."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        a, b, y = (in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B"),
                   out_desc_with_name(node, state, sdfg, "Y"))
        return _float_descs(a, b, y) and _matmul_plan(a.shape, b.shape) is not None

    @staticmethod
    def forward(node, state, sdfg):
        a, b = in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B")
        plan = _matmul_plan(a.shape, b.shape)
        bc = _b_is_constant(node, state, sdfg)

        def run(ins, outs):
            _launch_gemm(ins["A"], ins["B"], outs["Y"], plan, b_constant=bc)

        return KernelTasklet(node.label, run, kernels=("gemm",))


@op_implementation(op="Gemm", name="b200")
class B200Gemm(ONNXForward):
    """Gemm with alpha, beta * C and both transposes in one kernel (the reference needs up to three passes)."""
    @staticmethod
    def _c_mode(node, state, sdfg):
        if not _has_in(node, state, "C") or node.beta == 0:
            return "none"
        c = in_desc_with_name(node, state, sdfg, "C")
        y = out_desc_with_name(node, state, sdfg, "Y")
        # C is indexed by the trailing result indices and must match them exactly (:533-539)
        if len(c.shape) > len(y.shape) or tuple(c.shape) != tuple(y.shape[len(y.shape) - len(c.shape):]):
            raise ValueError('Could not broadcast dimensions from C to Y in ONNXGemm')
        return "bias" if len(c.shape) == 1 else "full"

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        a, b, y = (in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B"),
                   out_desc_with_name(node, state, sdfg, "Y"))
        return _float_descs(a, b, y) and len(a.shape) == 2 and len(b.shape) == 2

    @staticmethod
    def forward(node, state, sdfg):
        a, b = in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B")
        ta, tb = int(node.transA), int(node.transB)
        m, k = (a.shape[1], a.shape[0]) if ta else a.shape
        n = b.shape[0] if tb else b.shape[1]
        plan = dict(batch=1, m=m, k=k, n=n, a_batched=False, b_batched=False)
        mode = B200Gemm._c_mode(node, state, sdfg)
        alpha, beta = float(node.alpha), float(node.beta)
        bc = _b_is_constant(node, state, sdfg)

        def run(ins, outs):
            c = ins.get("C") if mode != "none" else None
            _launch_gemm(ins["A"], ins["B"], outs["Y"], plan, a_layout=ta, b_layout=tb, alpha=alpha, b_constant=bc,
                         bias=c if mode == "bias" else None, bias_scale=beta,
                         residual=c if mode == "full" else None, residual_scale=beta)

        return KernelTasklet(node.label, run, kernels=("gemm",))


def _parse_einsum(equation, shapes):
    """Recognises (batched) matrix products and pure permutations; returns a plan or None."""
    eq = equation.replace(" ", "")
    if "..." in eq or "->" not in eq:
        return None
    lhs, out = eq.split("->")
    terms = lhs.split(",")
    if len(terms) != len(shapes) or any(len(t) != len(s) for t, s in zip(terms, shapes)):
        return None
    if len(terms) == 1:
        t = terms[0]
        if sorted(t) != sorted(out) or len(set(t)) != len(t):
            return None
        return dict(kind="permute", perm=[t.index(c) for c in out])
    if len(terms) != 2:
        return None
    ta, tb = terms
    if len(set(ta)) != len(ta) or len(set(tb)) != len(tb) or len(set(out)) != len(out):
        return None
    size = {}
    for t, s in zip(terms, shapes):
        for c, e in zip(t, s):
            if size.setdefault(c, e) != e:
                return None
    nb = 0
    while nb < min(len(ta), len(tb), len(out)) and ta[nb] == tb[nb] == out[nb]:
        nb += 1
    batch = ta[:nb]
    ra, rb, ro = ta[nb:], tb[nb:], out[nb:]
    contracted = [c for c in ra if c in rb]
    if len(contracted) != 1 or contracted[0] in ro:
        return None
    kk = contracted[0]
    ml = [c for c in ra if c != kk]
    nl = [c for c in rb if c != kk]
    if ro != "".join(ml) + "".join(nl) or not ml or not nl:
        return None
    if ra == "".join(ml) + kk:
        a_layout = 0
    elif ra == kk + "".join(ml):
        a_layout = 1
    else:
        return None
    if rb == kk + "".join(nl):
        b_layout = 0
    elif rb == "".join(nl) + kk:
        b_layout = 1
    else:
        return None
    # leading letters of A that B lacks fold into M when nothing is batched ('zik,kj->zij')
    return dict(kind="gemm", batch=prod(size[c] for c in batch), m=prod(size[c] for c in ml),
                n=prod(size[c] for c in nl), k=size[kk], a_layout=a_layout, b_layout=b_layout,
                a_batched=nb > 0, b_batched=nb > 0)


@op_implementation(op="Einsum", name="b200")
class B200Einsum(ONNXForward):
    """Einsum equations that are (batched) matrix products or permutations."""
    @staticmethod
    def _plan(node, state, sdfg):
        edges = node.iter_inputs_in_onnx_order(state)
        descs = [sdfg.arrays[e.data.data] for e in edges]
        if not _float_descs(*descs) or node.equation is None:
            return None, edges
        return _parse_einsum(node.equation, [d.shape for d in descs]), edges

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        plan, _ = B200Einsum._plan(node, state, sdfg)
        return plan is not None

    @staticmethod
    def forward(node, state, sdfg):
        plan, edges = B200Einsum._plan(node, state, sdfg)
        conns = [e.dst_conn for e in edges]
        if plan["kind"] == "permute":
            perm = plan["perm"]

            def run_perm(ins, outs):
                K.transpose(ins[conns[0]], outs["Output"], perm)

            return KernelTasklet(node.label, run_perm, kernels=("transpose",))

        def run(ins, outs):
            _launch_gemm(ins[conns[0]], ins[conns[1]], outs["Output"], plan, a_layout=plan["a_layout"],
                         b_layout=plan["b_layout"])

        return KernelTasklet(node.label, run, kernels=("gemm",))


# ---------------------------------------------------------------------------------------------
# Softmax / LogSoftmax (pure_implementations.py:304-319, 649-656): opset <= 12 "coerce to 2-D"
# ---------------------------------------------------------------------------------------------
def _softmax_like(node, state, sdfg, log):
    x = in_desc_with_name(node, state, sdfg, "input")
    axis = _norm_axis(int(node.axis), len(x.shape))
    rows, cols = prod(x.shape[:axis]), prod(x.shape[axis:])

    def run(ins, outs):
        K.softmax(ins["input"], outs["output"], rows=rows, cols=cols, log=log)

    return KernelTasklet(node.label, run, kernels=("softmax",))


@op_implementation(op="Softmax", name="b200")
class B200Softmax(ONNXForward):
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        return _float_descs(in_desc_with_name(node, state, sdfg, "input"), out_desc_with_name(node, state, sdfg, "output"))

    @staticmethod
    def forward(node, state, sdfg):
        return _softmax_like(node, state, sdfg, False)


@op_implementation(op="LogSoftmax", name="b200")
class B200LogSoftmax(ONNXForward):
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        return _float_descs(in_desc_with_name(node, state, sdfg, "input"), out_desc_with_name(node, state, sdfg, "output"))

    @staticmethod
    def forward(node, state, sdfg):
        return _softmax_like(node, state, sdfg, True)


# ---------------------------------------------------------------------------------------------
# Element-wise (pure_implementations.py:24-108, 283-291, 556-568, 736-743)
# ---------------------------------------------------------------------------------------------
def _register_binary(op, code, a="A", b="B", c="C"):
    def can(node, state, sdfg):
        da, db, dc = (in_desc_with_name(node, state, sdfg, a), in_desc_with_name(node, state, sdfg, b),
                      out_desc_with_name(node, state, sdfg, c))
        if not _float_descs(da, db, dc) or len(dc.shape) > 6:
            return False
        try:
            return tuple(torch.broadcast_shapes(da.shape, db.shape)) == tuple(dc.shape)
        except RuntimeError:
            return False

    def fwd(node, state, sdfg):
        def run(ins, outs):
            K.binary(ins[a], ins[b], outs[c], code)

        return KernelTasklet(node.label, run, kernels=("binary",))

    cls = type("B200" + op, (ONNXForward, ), dict(forward_can_be_applied=staticmethod(can), forward=staticmethod(fwd),
                                                 __doc__="Numpy-broadcast {}.".format(op)))
    return op_implementation(op=op, name="b200")(cls)


B200Add = _register_binary("Add", L.BIN_ADD)
B200Sub = _register_binary("Sub", L.BIN_SUB)
B200Mul = _register_binary("Mul", L.BIN_MUL)
B200Div = _register_binary("Div", L.BIN_DIV)
B200Pow = _register_binary("Pow", L.BIN_POW, "X", "Y", "Z")


def _register_unary(op, code, i="X", o="Y", params=None):
    def can(node, state, sdfg):
        return _float_descs(in_desc_with_name(node, state, sdfg, i), out_desc_with_name(node, state, sdfg, o))

    def fwd(node, state, sdfg):
        p0, p1 = params(node) if params else (0.0, 0.0)

        def run(ins, outs):
            K.unary(ins[i], outs[o], code, p0, p1)

        return KernelTasklet(node.label, run, kernels=("unary",))

    cls = type("B200" + op, (ONNXForward, ), dict(forward_can_be_applied=staticmethod(can), forward=staticmethod(fwd),
                                                 __doc__="Element-wise {}.".format(op)))
    return op_implementation(op=op, name="b200")(cls)


B200Sqrt = _register_unary("Sqrt", L.UN_SQRT)
B200Relu = _register_unary("Relu", L.UN_RELU)
B200Sigmoid = _register_unary("Sigmoid", L.UN_SIGMOID)
B200Reciprocal = _register_unary("Reciprocal", L.UN_RECIPROCAL)
B200Softplus = _register_unary("Softplus", L.UN_SOFTPLUS)
B200LeakyRelu = _register_unary("LeakyRelu", L.UN_LEAKYRELU, params=lambda n: (float(n.alpha), 0.0))
B200Erf = _register_unary("Erf", L.UN_ERF, "input", "output")
B200Exp = _register_unary("Exp", L.UN_EXP, "input", "output")
B200Log = _register_unary("Log", L.UN_LOG, "input", "output")
B200Tanh = _register_unary("Tanh", L.UN_TANH, "input", "output")
B200Identity = _register_unary("Identity", L.UN_COPY, "input", "output")
B200Gelu = _register_unary("Gelu", L.UN_GELU)
B200Swish = _register_unary("Swish", L.UN_SWISH)
B200Neg = _register_unary("Neg", L.UN_NEG)


def _constant_value(sdfg, state, node, conn):
    for e in state.in_edges_by_connector(node, conn):
        t = sdfg.constants.get(e.data.data)
        if t is not None and t.numel() == 1:
            return float(t.reshape(-1)[0])
    return None


@op_implementation(op="Clip", name="b200")
class B200Clip(ONNXForward):
    """Clip with constant bounds, like the reference (pure_implementations.py:44-73)."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        if not _float_descs(in_desc_with_name(node, state, sdfg, "input"), out_desc_with_name(node, state, sdfg, "output")):
            return False
        return all(not _has_in(node, state, c) or _constant_value(sdfg, state, node, c) is not None for c in ("min", "max"))

    @staticmethod
    def forward(node, state, sdfg):
        lo = _constant_value(sdfg, state, node, "min") if _has_in(node, state, "min") else -3.0e38
        hi = _constant_value(sdfg, state, node, "max") if _has_in(node, state, "max") else 3.0e38

        def run(ins, outs):
            K.unary(ins["input"], outs["output"], L.UN_CLIP, lo, hi)

        return KernelTasklet(node.label, run, kernels=("unary",))


@op_implementation(op="Cast", name="b200")
class B200Cast(ONNXForward):
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        i, o = in_desc_with_name(node, state, sdfg, "input"), out_desc_with_name(node, state, sdfg, "output")
        return i.dtype in L.CAST_CODES and o.dtype in L.CAST_CODES and i.total_size() == o.total_size()

    @staticmethod
    def forward(node, state, sdfg):
        def run(ins, outs):
            K.cast(ins["input"], outs["output"])

        return KernelTasklet(node.label, run, kernels=("cast",))


@op_implementation(op="Sum", name="b200")
class B200Sum(ONNXForward):
    """Variadic Sum of same-shape tensors (the reference's precondition, pure_implementations.py:584-604)."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        descs = [sdfg.arrays[e.data.data] for e in node.iter_inputs_in_onnx_order(state)]
        out = out_desc_with_name(node, state, sdfg, "sum")
        return _float_descs(*descs, out) and all(tuple(d.shape) == tuple(out.shape) for d in descs)

    @staticmethod
    def forward(node, state, sdfg):
        conns = [e.dst_conn for e in node.iter_inputs_in_onnx_order(state)]

        def run(ins, outs):
            y = outs["sum"]
            if len(conns) == 1:
                K.unary(ins[conns[0]], y, L.UN_COPY)
                return
            K.binary(ins[conns[0]], ins[conns[1]], y, L.BIN_ADD)
            for c in conns[2:]:
                K.binary(y, ins[c], y, L.BIN_ADD)

        return KernelTasklet(node.label, run, kernels=("binary",))


# ---------------------------------------------------------------------------------------------
# Reductions (pure_implementations.py:101-103, 294-306)
# ---------------------------------------------------------------------------------------------
def _reduce_groups(shape, axes):
    """Splits the reduced axes into runs of adjacent axes, last run first; each run is one launch."""
    rank = len(shape)
    axes = sorted({_norm_axis(int(a), rank) for a in axes}) if axes is not None else list(range(rank))
    runs, cur = [], []
    for a in axes:
        if cur and a != cur[-1] + 1:
            runs.append(cur)
            cur = []
        cur.append(a)
    if cur:
        runs.append(cur)
    return list(reversed(runs))


def _add_scratch(node, state, sdfg, tag, shape, dtype):
    """Declares a transient of the SDFG as scratch of ``node`` and hangs it on an extra output connector, so that it is
    allocated with the other transients when the SDFG is compiled -- never inside a launch (which may be under CUDA-graph
    capture).  Returns the connector name under which the tasklet finds the tensor in ``outs``."""
    base, i = "{}_{}".format(node.label, tag), 0
    name = base
    while name in sdfg.arrays:
        i += 1
        name = "{}_{}".format(base, i)
    sdfg.add_transient(name, tuple(shape), dtype)
    conn = "__scratch_" + tag
    state.add_edge(node, conn, state.add_write(name), None, sdfg.make_array_memlet(name))
    return conn


def _register_reduce(op, code):
    def can(node, state, sdfg):
        return _float_descs(in_desc_with_name(node, state, sdfg, "data"), out_desc_with_name(node, state, sdfg, "reduced"))

    def fwd(node, state, sdfg):
        shape = list(in_desc_with_name(node, state, sdfg, "data").shape)
        runs = _reduce_groups(shape, node.axes)
        steps, cur = [], list(shape)
        for run_axes in runs:
            lo, hi = run_axes[0], run_axes[-1]
            steps.append((prod(cur[:lo]), prod(cur[lo:hi + 1]), prod(cur[hi + 1:])))
            cur = cur[:lo] + cur[hi + 1:]
        dtype = in_desc_with_name(node, state, sdfg, "data").dtype
        temps = {i: _add_scratch(node, state, sdfg, "partial%d" % i, (outer * inner, ), dtype)
                 for i, (outer, _, inner) in enumerate(steps[:-1])}

        def run(ins, outs):
            src, dst = ins["data"], outs["reduced"]
            if not steps:
                K.unary(src, dst, L.UN_COPY)
                return
            for i, (outer, red, inner) in enumerate(steps):
                tgt = dst if i == len(steps) - 1 else outs[temps[i]]
                K.reduce(src, tgt, op=code, outer=outer, red=red, inner=inner)
                src = tgt

        return KernelTasklet(node.label, run, kernels=("reduce",))

    cls = type("B200" + op, (ONNXForward, ), dict(forward_can_be_applied=staticmethod(can), forward=staticmethod(fwd),
                                                 __doc__="{} over node.axes.".format(op)))
    return op_implementation(op=op, name="b200")(cls)


B200ReduceSum = _register_reduce("ReduceSum", L.RED_SUM)
B200ReduceMean = _register_reduce("ReduceMean", L.RED_MEAN)
B200ReduceMax = _register_reduce("ReduceMax", L.RED_MAX)
B200ReduceMin = _register_reduce("ReduceMin", L.RED_MIN)


@op_implementation(op="GlobalAveragePool", name="b200")
class B200GlobalAveragePool(ONNXForward):
    """Mean over H, W (img_op_implementations.py:415-526): one warp per (image, channel) plane."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x = in_desc_with_name(node, state, sdfg, "X")
        return _float_descs(x, out_desc_with_name(node, state, sdfg, "Y")) and len(x.shape) == 4

    @staticmethod
    def forward(node, state, sdfg):
        n, c, h, w = in_desc_with_name(node, state, sdfg, "X").shape

        def run(ins, outs):
            K.reduce(ins["X"], outs["Y"], op=L.RED_MEAN, outer=n * c, red=h * w, inner=1)

        return KernelTasklet(node.label, run, kernels=("reduce",))


# ---------------------------------------------------------------------------------------------
# Data movement (pure_implementations.py:322-326, 571-581, 746-778, 1016-1026)
# ---------------------------------------------------------------------------------------------
@op_implementation(op="Transpose", name="b200")
class B200Transpose(ONNXForward):
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        d = in_desc_with_name(node, state, sdfg, "data")
        return d.dtype.itemsize in (2, 4) and 1 <= len(d.shape) <= 6

    @staticmethod
    def forward(node, state, sdfg):
        rank = len(in_desc_with_name(node, state, sdfg, "data").shape)
        perm = list(node.perm) if node.perm is not None else list(reversed(range(rank)))

        def run(ins, outs):
            K.transpose(ins["data"], outs["transposed"], perm)

        return KernelTasklet(node.label, run, kernels=("transpose",))


def _register_copy(op, i, o):
    """Reshape-like nodes copy their input into the output descriptor's shape, as the reference does."""
    def can(node, state, sdfg):
        a, b = in_desc_with_name(node, state, sdfg, i), out_desc_with_name(node, state, sdfg, o)
        return a.dtype == b.dtype and a.total_size() == b.total_size() and (
            a.dtype in FLOAT_TYPES or torch.empty((), dtype=a.dtype).element_size() in (1, 2, 4, 8))

    def fwd(node, state, sdfg):
        if in_desc_with_name(node, state, sdfg, i).dtype in FLOAT_TYPES:
            def run(ins, outs):
                K.unary(ins[i], outs[o], L.UN_COPY)

            return KernelTasklet(node.label, run, kernels=("unary",))

        def run_bytes(ins, outs):  # index and mask tensors (int64, bool): a plain copy of the bytes
            K.strided_copy(ins[i].reshape(-1), outs[o].reshape(-1))

        return KernelTasklet(node.label, run_bytes, kernels=("strided_copy",))

    cls = type("B200" + op, (ONNXForward, ), dict(forward_can_be_applied=staticmethod(can), forward=staticmethod(fwd),
                                                 __doc__="{} as a flat copy.".format(op)))
    return op_implementation(op=op, name="b200")(cls)


B200Reshape = _register_copy("Reshape", "data", "reshaped")
B200Flatten = _register_copy("Flatten", "input", "output")
B200Unsqueeze = _register_copy("Unsqueeze", "data", "expanded")
B200Squeeze = _register_copy("Squeeze", "data", "squeezed")


# ---------------------------------------------------------------------------------------------
# Conv (img_op_implementations.py:164-330, cudnn_implementations.py:123-410)
# ---------------------------------------------------------------------------------------------
def _conv_geometry(node, x, w):
    kh, kw = w.shape[2:]
    strides = list(node.strides) if node.strides else [1, 1]
    dil = list(node.dilations) if node.dilations else [1, 1]
    pads = list(node.pads) if node.pads else [0, 0, 0, 0]
    return strides, dil, pads, int(node.group)


def _conv_can(node, state, sdfg):
    x, w, y = (in_desc_with_name(node, state, sdfg, "X"), in_desc_with_name(node, state, sdfg, "W"),
               out_desc_with_name(node, state, sdfg, "Y"))
    if not _float_descs(x, w, y) or len(x.shape) != 4 or len(w.shape) != 4:
        return False
    if getattr(node, "auto_pad", "NOTSET") not in ("NOTSET", "VALID"):
        return False
    g = int(node.group)
    return x.shape[1] % g == 0 and w.shape[0] % g == 0 and w.shape[1] == x.shape[1] // g


def _prepacked_conv_weights(node, state, sdfg, x, strides, pads, dil, group, gate):
    """Weights (and bias) that are constants of the SDFG are prepared for the tensor-core kernels once, here, instead
    of by a small kernel at every call (``b200ml_conv_prepack``).  Returns the packed tensor or None (no device, the
    weights arrive at run time, or the convolution runs on a kernel that takes them as they are)."""
    if not torch.cuda.is_available() or not _b_is_constant(node, state, sdfg, "W"):
        return None
    if _has_in(node, state, "B") and not _b_is_constant(node, state, sdfg, "B"):
        return None
    dev = torch.device("cuda", torch.cuda.current_device())  # calls on another device ignore the packed copy
    tensors = {}
    for conn in ("W", "B"):
        for e in state.in_edges_by_connector(node, conn):
            t = sdfg.constants[e.data.data]
            if not t.is_cuda:  # a copy for the packing kernel only; the SDFG's own constant moves with its first call
                t = t.to(dev)
            tensors[conn] = t.contiguous()
    w = tensors["W"]
    if w.dtype != torch.float32 or not w.is_contiguous():
        return None
    return K.conv_prepack(tuple(x.shape), w, bias=tensors.get("B"), strides=strides, pads=pads, dilations=dil, group=group, gate=gate)


@op_implementation(op="Conv", name="b200")
class B200Conv(ONNXForward):
    """2-D convolution with strides, pads, dilations and groups (the reference's pure Conv rejects all four)."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        return _conv_can(node, state, sdfg)

    @staticmethod
    def forward(node, state, sdfg):
        x, w = in_desc_with_name(node, state, sdfg, "X"), in_desc_with_name(node, state, sdfg, "W")
        strides, dil, pads, group = _conv_geometry(node, x, w)
        packed = _prepacked_conv_weights(node, state, sdfg, x, strides, pads, dil, group, False)

        def run(ins, outs):
            xt = ins["X"]
            K.conv2d(xt, ins["W"], outs["Y"], bias=ins.get("B"), strides=strides, pads=pads, dilations=dil,
                     group=group, packed_weight=packed if packed is not None and packed.device == xt.device else None)

        return KernelTasklet(node.label, run, kernels=("conv2d",))


_ACT = {"": 0, "Relu": L.EPI_RELU, "Gelu": L.EPI_GELU, "Swish": L.EPI_SWISH}


@op_implementation(op="BatchNormalization", name="b200")
class B200BatchNormalization(ONNXForward):
    """Inference BatchNormalization with constant statistics: ``Y = a * X + b`` per channel, ``a = scale / sqrt(var +
    eps)``, ``b = B - mean * a``, run as a depthwise 1x1 convolution (one read of X, one write of Y).  The reference's
    pure and cuDNN expansions are the training form (``img_op_implementations.py:333-393``,
    ``cudnn_implementations.py:413-``), which this library does not implement."""

    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        from daceml_b200.transformation.patterns import batchnorm_affine
        x, y = in_desc_with_name(node, state, sdfg, "X"), out_desc_with_name(node, state, sdfg, "Y")
        return (_float_descs(x, y) and 2 <= len(x.shape) <= 4 and tuple(x.shape) == tuple(y.shape)
                and batchnorm_affine(sdfg, state, node) is not None)

    @staticmethod
    def forward(node, state, sdfg):
        from daceml_b200.transformation.patterns import batchnorm_affine
        a, b = batchnorm_affine(sdfg, state, node)
        x = in_desc_with_name(node, state, sdfg, "X")
        shape4 = tuple(x.shape) + (1, ) * (4 - len(x.shape))
        cache = {}

        def run(ins, outs):
            t = ins["X"]
            key = (t.device, t.dtype)
            if key not in cache:
                cache[key] = (a.reshape(-1, 1, 1, 1).to(t.dtype).to(t.device).contiguous(), b.to(t.dtype).to(t.device).contiguous())
            w, bias = cache[key]
            K.conv2d(t.view(shape4), w, outs["Y"].view(shape4), bias=bias, group=shape4[1])

        return KernelTasklet(node.label, run, kernels=("conv2d",))


@op_implementation(op="FusedConv", name="b200")
class B200FusedConv(ONNXForward):
    """Conv + bias + activation, with a squeeze-excite gate on the input, a residual add and the
    GlobalAveragePool of the result folded in."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        return _conv_can(node, state, sdfg) and node.activation in _ACT

    @staticmethod
    def forward(node, state, sdfg):
        x, w = in_desc_with_name(node, state, sdfg, "X"), in_desc_with_name(node, state, sdfg, "W")
        strides, dil, pads, group = _conv_geometry(node, x, w)
        act = _ACT[node.activation]
        packed = _prepacked_conv_weights(node, state, sdfg, x, strides, pads, dil, group, _has_in(node, state, "Gate"))

        def run(ins, outs):
            xt = ins["X"]
            K.conv2d(xt, ins["W"], outs["Y"], bias=ins.get("B"), strides=strides, pads=pads, dilations=dil,
                     group=group, act=act, gate=ins.get("Gate"), residual=ins.get("Residual"),
                     pool_mean=outs.get("Pool"), packed_weight=packed if packed is not None and packed.device == xt.device else None)

        return KernelTasklet(node.label, run, kernels=("conv2d",))


@op_implementation(op="SqueezeExcite", name="b200")
class B200SqueezeExcite(ONNXForward):
    """sigmoid(W2 . swish(W1 . pooled + b1) + b2): both 1x1 convolutions of the gate in one launch."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x = in_desc_with_name(node, state, sdfg, "X")
        return x.dtype in FLOAT_TYPES and len(x.shape) == 4 and x.shape[2] == 1 and x.shape[3] == 1

    @staticmethod
    def forward(node, state, sdfg):
        def run(ins, outs):
            K.se_gate(ins["X"], ins["W1"], ins.get("B1"), ins["W2"], ins.get("B2"), outs["Y"])

        return KernelTasklet(node.label, run, kernels=("se_gate",))


# ---------------------------------------------------------------------------------------------
# Fused transformer operators
# ---------------------------------------------------------------------------------------------
@op_implementation(op="LayerNormalization", name="b200")
class B200LayerNormalization(ONNXForward):
    """The ReduceMean/Sub/Pow/ReduceMean/Add/Sqrt/Div/Mul/Add chain (and the residual Add before it) in one pass."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        x = in_desc_with_name(node, state, sdfg, "X")
        return x.dtype in FLOAT_TYPES and _norm_axis(int(node.axis), len(x.shape)) == len(x.shape) - 1

    @staticmethod
    def forward(node, state, sdfg):
        eps = float(node.epsilon)

        def run(ins, outs):
            K.layernorm(ins["X"], outs["Y"], gamma=ins.get("Scale"), beta=ins.get("B"), residual=ins.get("Residual"),
                        eps=eps)

        return KernelTasklet(node.label, run, kernels=("layernorm",))


@op_implementation(op="FusedMatMul", name="b200")
class B200FusedMatMul(ONNXForward):
    """MatMul with the bias Add, the activation chain and the residual Add in the GEMM epilogue."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        a, b = in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B")
        return _float_descs(a, b) and len(b.shape) == 2 and len(a.shape) >= 2 and node.activation in _ACT

    @staticmethod
    def forward(node, state, sdfg):
        a, b = in_desc_with_name(node, state, sdfg, "A"), in_desc_with_name(node, state, sdfg, "B")
        tb = int(node.transB)
        k = a.shape[-1]
        n = b.shape[0] if tb else b.shape[1]
        plan = dict(batch=1, m=prod(a.shape[:-1]), k=k, n=n, a_batched=False, b_batched=False)
        act, alpha = _ACT[node.activation], float(node.alpha)
        bc = _b_is_constant(node, state, sdfg)
        if node.ln_epsilon is None:

            def run(ins, outs):
                _launch_gemm(ins["A"], ins["B"], outs["Y"], plan, b_layout=tb, alpha=alpha, bias=ins.get("Bias"),
                             residual=ins.get("Residual"), act=act, b_constant=bc)

            return KernelTasklet(node.label, run, kernels=("gemm",))

        # LayerNorm of the result: inside the GEMM epilogue where the fused kernel covers the shape (fp16, N a
        # multiple of 256 up to 1024), else as a second launch on a pre-normalisation buffer.
        eps = float(node.ln_epsilon)
        fusable = a.dtype == torch.float16 and n in (256, 512, 1024) and k % 8 == 0 and act in (0, L.EPI_RELU)
        if fusable:

            def run_fused(ins, outs):
                _launch_gemm(ins["A"], ins["B"], outs["Y"], plan, b_layout=tb, alpha=alpha, bias=ins.get("Bias"),
                             residual=ins.get("Residual"), act=act, ln=(ins.get("LnScale"), ins.get("LnBias"), eps),
                             b_constant=bc)

            return KernelTasklet(node.label, run_fused, kernels=("gemm_layernorm",))
        y_desc = out_desc_with_name(node, state, sdfg, "Y")
        pre = _add_scratch(node, state, sdfg, "prenorm", y_desc.shape, y_desc.dtype)

        def run_split(ins, outs):
            y, tmp = outs["Y"], outs[pre]
            _launch_gemm(ins["A"], ins["B"], tmp, plan, b_layout=tb, alpha=alpha, bias=ins.get("Bias"),
                         residual=ins.get("Residual"), act=act, b_constant=bc)
            K.layernorm(tmp, y, gamma=ins.get("LnScale"), beta=ins.get("LnBias"), eps=eps)

        return KernelTasklet(node.label, run_split, kernels=("gemm", "layernorm"))


@op_implementation(op="Attention", name="b200")
class B200Attention(ONNXForward):
    """softmax(scale * Q K^T + mask) V without materialising the scores.

    Q, K, V are [B, S, heads * d]; when K and V are not connected, Q is the packed [B, S, 3 * heads * d]
    output of one QKV projection and the heads are addressed inside it by strides."""
    @staticmethod
    def forward_can_be_applied(node, state, sdfg):
        q = in_desc_with_name(node, state, sdfg, "Q")
        if q.dtype != torch.float16 or len(q.shape) != 3:
            return False
        packed = not _has_in(node, state, "K")
        hidden = q.shape[2] // 3 if packed else q.shape[2]
        return hidden % int(node.num_heads) == 0 and hidden // int(node.num_heads) == 64

    @staticmethod
    def forward(node, state, sdfg):
        q = in_desc_with_name(node, state, sdfg, "Q")
        heads = int(node.num_heads)
        packed = not _has_in(node, state, "K")
        hidden = q.shape[2] // 3 if packed else q.shape[2]
        d = hidden // heads
        scale = float(node.scale) if node.scale is not None else 1.0 / math.sqrt(d)

        def heads_view(t, offset, width):
            b, s, _ = t.shape
            return t.as_strided((b, heads, s, d), (s * width, d, width, 1), t.storage_offset() + offset)

        def run(ins, outs):
            if packed:
                qkv = ins["Q"]
                w = 3 * hidden
                qv, kv, vv = heads_view(qkv, 0, w), heads_view(qkv, hidden, w), heads_view(qkv, 2 * hidden, w)
            else:
                qv, kv, vv = (heads_view(ins[c], 0, hidden) for c in ("Q", "K", "V"))
            K.attention(qv, kv, vv, heads_view(outs["Y"], 0, hidden), scale=scale, mask=ins.get("Mask"))

        return KernelTasklet(node.label, run, kernels=("attention",))
