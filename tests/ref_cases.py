"""The fixtures produced from the reference's own source (tests/golden/ref_pure_expansions.*) and the two ways the
tests replay a case: through the CPU oracle (``oracle_outputs``) and through the donnx frontend on the GPU
(``frontend_outputs``)."""
import functools
import json
import os

import numpy as np

from oracle import ops

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
with open(os.path.join(GOLD, "ref_pure_expansions.json")) as _f:
    REF_CASES = json.load(_f)["cases"]

# pure data movement and selection: compared bit for bit
BIT_EXACT_OPS = {"Identity", "Expand", "Where", "Transpose", "Reshape", "Flatten", "Unsqueeze", "Shape", "Cast", "Gather",
                 "Split", "Slice", "Relu", "Clip", "ReduceMax", "ReduceMin"}


@functools.lru_cache(maxsize=1)
def ref_arrays():
    with np.load(os.path.join(GOLD, "ref_pure_expansions.npz")) as z:
        return {k: z[k] for k in z.files}


def case_inputs(case, arrays):
    return {k: arrays["%s:%s" % (case["case"], k)] for k in case["inputs"]}


_UNARY = {"Log": ops.log, "Exp": ops.exp, "Sqrt": ops.sqrt, "Tanh": ops.tanh, "Erf": ops.erf, "Relu": ops.relu,
          "Sigmoid": ops.sigmoid, "Softplus": ops.softplus, "Reciprocal": ops.reciprocal, "Identity": ops.identity}
_BINARY = {"Add": ops.add, "Sub": ops.sub, "Mul": ops.mul, "Div": ops.div, "Pow": ops.pow_}
_REDUCE = {"ReduceSum": ops.reduce_sum, "ReduceMean": ops.reduce_mean, "ReduceMax": ops.reduce_max, "ReduceMin": ops.reduce_min}


def oracle_outputs(case, arrays):
    """The case's outputs according to ``oracle/ops.py``: connector name -> array."""
    op, at, x = case["op"], case["attrs"], case_inputs(case, arrays)
    out = case["outputs"][0]
    first = next(iter(x.values()))
    if op in _UNARY:
        return {out: _UNARY[op](first)}
    if op == "LeakyRelu":
        return {out: ops.leaky_relu(first, at["alpha"])}
    if op == "Clip":
        return {out: ops.clip(x["input"], x["min"], x["max"])}
    if op == "Expand":
        return {out: ops.expand(x["input"], x["shape"])}
    if op in _BINARY:
        a, b = list(x.values())
        return {out: _BINARY[op](a, b)}
    if op == "Where":
        return {out: ops.where(x["condition"], x["X"], x["Y"])}
    if op == "Sum":
        vals = list(x.values())
        acc = vals[0]
        for v in vals[1:]:
            acc = ops.add(acc, v)
        return {out: acc}
    if op in _REDUCE:
        r = _REDUCE[op](x["data"], at["axes"], at["keepdims"])
        return {out: r.reshape(arrays["%s:%s" % (case["case"], out)].shape)}  # a full reduction is stored as [1]
    if op == "GlobalAveragePool":
        return {out: ops.global_average_pool(x["X"])}
    if op == "Softmax":
        return {out: ops.softmax(x["input"], at["axis"])}
    if op == "LogSoftmax":
        return {out: ops.log_softmax(x["input"], at["axis"])}
    if op == "Transpose":
        return {out: ops.transpose(x["data"], at["perm"])}
    if op == "Reshape":
        return {out: ops.reshape(x["data"], [int(s) for s in x["shape"]])}
    if op == "Flatten":
        return {out: ops.flatten(x["input"], at["axis"])}
    if op == "Unsqueeze":
        return {out: ops.unsqueeze(x["data"], at["axes"])}
    if op == "Shape":
        return {out: ops.shape(x["data"])}
    if op == "Cast":
        return {out: ops.cast(x["input"], np.dtype(at["to"]))}
    if op == "Gather":
        return {out: ops.gather(x["data"], x["indices"], at["axis"])}
    if op == "Split":
        parts = ops.split(x["input"], at["axis"], at["split"])
        return {"outputs__%d" % i: p for i, p in enumerate(parts)}
    if op == "Slice":
        return {out: ops.slice_(x["data"], x["starts"], x["ends"], x["axes"], x["steps"])}
    if op == "MatMul":
        return {out: ops.matmul(x["A"], x["B"])}
    if op == "Gemm":
        return {out: ops.gemm(x["A"], x["B"], x.get("C"), at["alpha"], at["beta"], at["transA"], at["transB"])}
    if op == "Einsum":
        ins = [x[k] for k in sorted(x)]
        return {out: ops.einsum(at["equation"], *ins, acc_dtype=ins[0].dtype.type)}
    if op == "Conv":
        return {out: ops.conv2d(x["X"], x["W"], x.get("B"))}
    raise KeyError(op)


def _contig(a):
    """A C-contiguous copy that keeps a 0-d array 0-d (np.ascontiguousarray would make it 1-d)."""
    return np.array(a, copy=True, order="C")


def frontend_outputs(case, arrays, donnx, torch):
    """The case's outputs from the CUDA path: ``donnx.ONNX<Op>(connector=tensor, ..., attribute=value)`` with
    device tensors, as a user of the frontend calls it (index-like parameters stay on the host, where the frontend
    binds them as constants; a node with floating-point constants -- Clip's bounds -- is built through the SDFG API,
    as an importer would).  float64 cases run in float32.  Returns connector name -> (got, want) numpy arrays."""
    from daceml_b200 import sdfg as sd
    at = {k: v for k, v in case["attrs"].items() if v is not None}
    if case["op"] == "Cast":
        at["to"] = {"float32": 1, "int32": 6, "int64": 7}[at["to"]]  # ONNX TensorProto data types
    if case["op"] == "Conv":
        at = {k: v for k, v in at.items() if k in ("group", "dilations", "pads", "strides")}
    if case["implementation"] != "pure":
        at = dict(at)
    narrow = lambda a: a.astype(np.float32) if a.dtype == np.float64 else a
    host_params = set(case["constants"]) | ({"shape"} if case["op"] in ("Reshape", "Expand") else set())
    ins = {k: narrow(v) for k, v in case_inputs(case, arrays).items()}
    want = {k: narrow(arrays["%s:%s" % (case["case"], k)]) for k in case["outputs"]}
    outs = {k: torch.empty(w.shape, dtype=torch.from_numpy(np.empty(0, w.dtype)).dtype, device="cuda") for k, w in want.items()}
    float_constants = [k for k in host_params if np.issubdtype(ins[k].dtype, np.floating)]
    if float_constants:
        g = sd.SDFG("case_" + case["case"])
        st = g.add_state()
        node = getattr(donnx, "ONNX" + case["op"])(case["op"], **at)
        st.add_node(node)
        call = {}
        for k, v in ins.items():
            if k in host_params:
                g.add_constant("arr_" + k, torch.from_numpy(_contig(v)))
            else:
                g.add_array("arr_" + k, v.shape, v.dtype)
                call["arr_" + k] = torch.from_numpy(_contig(v)).cuda()
            st.add_edge(st.add_read("arr_" + k), None, node, k, g.make_array_memlet("arr_" + k))
        for k, o in outs.items():
            g.add_array("arr_" + k, o.shape, o.dtype)
            call["arr_" + k] = o
            st.add_edge(node, k, st.add_write("arr_" + k), None, g.make_array_memlet("arr_" + k))
        g.compile()(**call)
    else:
        kw = {k: (_contig(v) if k in host_params else torch.from_numpy(_contig(v)).cuda()) for k, v in ins.items()}
        kw.update(outs)
        getattr(donnx, "ONNX" + case["op"])(**kw, **at)
    torch.cuda.synchronize()
    return {k: (outs[k].cpu().numpy(), want[k]) for k in outs}
