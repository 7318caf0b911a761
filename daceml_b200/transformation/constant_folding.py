"""Constant folding: nodes whose inputs are all known at build time are evaluated once on the host.

The analogue of the reference's ``ConstantFolding`` transformation
(``daceml/transformation/constant_folding.py:50-197``), which evaluates such nodes with ONNX Runtime
and turns their outputs into weights.  Here the evaluation is a small table of torch functions over
the constants (weights live in ``sdfg.constants``); ``Shape`` of any array also folds, since every
array has a static shape.  This removes the weight ``Transpose`` nodes and the
``Shape -> Gather -> Unsqueeze -> Concat -> Reshape`` arithmetic an export without exporter-side
folding contains.
"""
import math

import torch

import daceml_b200.onnx as donnx
from daceml_b200 import sdfg as sd
from . import patterns as P


def _axes(node):
    return [int(a) for a in (node.axes or [])]


def _reshape(data, shape):
    shape = [int(s) for s in shape.tolist()]
    shape = [data.shape[i] if s == 0 else s for i, s in enumerate(shape)]  # opset 5-13: 0 copies the input extent
    return data.reshape(shape)


def _unsqueeze(data, axes):
    rank = data.dim() + len(axes)
    for a in sorted(a % rank for a in axes):
        data = data.unsqueeze(a)
    return data


def _squeeze(data, axes):
    if not axes:
        return data.squeeze()
    for a in sorted((a % data.dim() for a in axes), reverse=True):
        data = data.squeeze(a)
    return data


def _slice(data, starts, ends, axes=None, steps=None):
    starts, ends = starts.tolist(), ends.tolist()
    axes = axes.tolist() if axes is not None else list(range(len(starts)))
    steps = steps.tolist() if steps is not None else [1] * len(starts)
    index = [slice(None)] * data.dim()
    for s, e, a, st in zip(starts, ends, axes, steps):
        if st <= 0:
            raise NotImplementedError("Slice with a non-positive step")
        n = data.shape[a]
        s = max(0, min(n, s + n if s < 0 else s))
        e = max(0, min(n, e + n if e < 0 else e))
        index[a] = slice(s, e, st)
    return data[tuple(index)]


def _gather(data, indices, axis):
    axis %= data.dim()
    flat = torch.index_select(data, axis, indices.reshape(-1).long() % data.shape[axis])
    return flat.reshape(tuple(data.shape[:axis]) + tuple(indices.shape) + tuple(data.shape[axis + 1:]))


def _cast(data, to):
    from daceml_b200.onnx.converters import onnx_tensor_type_to_torch
    return data.to(onnx_tensor_type_to_torch(int(to)))


def _binary(fn):
    return lambda n, i: fn(i["A"], i["B"])


# op -> function(node, {connector: tensor}) -> tensor
_EVAL = {
    "Transpose": lambda n, i: i["data"].permute(*(n.perm or list(reversed(range(i["data"].dim()))))),
    "Reshape": lambda n, i: _reshape(i["data"], i["shape"]),
    "Flatten": lambda n, i: i["input"].reshape(math.prod(i["input"].shape[:int(n.axis)]), -1),
    "Unsqueeze": lambda n, i: _unsqueeze(i["data"], _axes(n)),
    "Squeeze": lambda n, i: _squeeze(i["data"], _axes(n)),
    "Identity": lambda n, i: i["input"],
    "Cast": lambda n, i: _cast(i["input"], n.to),
    "Gather": lambda n, i: _gather(i["data"], i["indices"], int(n.axis)),
    "Concat": lambda n, i: torch.cat([i[k] for k in sorted(i, key=lambda c: int(c.split("__")[1]))], int(n.axis)),
    "Slice": lambda n, i: _slice(i["data"], i["starts"], i["ends"], i.get("axes"), i.get("steps")),
    "ConstantOfShape": lambda n, i: torch.full([int(s) for s in i["input"].tolist()],
                                               (n.value.reshape(-1)[0].item() if n.value is not None else 0.0),
                                               dtype=(n.value.dtype if n.value is not None else torch.float32)),
    "Neg": lambda n, i: -i["X"],
    "Sqrt": lambda n, i: torch.sqrt(i["X"]),
    "Add": _binary(torch.add), "Sub": _binary(torch.sub), "Mul": _binary(torch.mul),
    "Div": lambda n, i: (torch.div(i["A"], i["B"], rounding_mode="trunc") if not i["A"].is_floating_point() else i["A"] / i["B"]),
}


def _split(node, ins):
    x = ins["input"]
    axis = int(node.axis) % x.dim()
    return torch.split(x, [int(n) for n in node.split] if node.split else x.shape[axis] // max(len(node.out_connectors), 1), axis)


def _fold_split(sdfg, state, node):
    """Split of a constant: every output becomes a constant (outputs are ``outputs__i`` in order)."""
    x = sdfg.constants.get(P._in(state, node, "input"))
    outs = sorted(state.out_edges(node), key=lambda e: int(e.src_conn.split("__")[1]))
    if x is None or any(not sdfg.arrays[e.data.data].transient for e in outs):
        return False
    parts = _split(node, dict(input=x))
    if len(parts) != len(outs) or any(tuple(p.shape) != tuple(sdfg.arrays[e.data.data].shape) for p, e in zip(parts, outs)):
        return False
    state.remove_node(node)
    for p, e in zip(parts, outs):
        name = e.data.data
        dtype = sdfg.arrays[name].dtype
        del sdfg.arrays[name]
        sdfg.add_constant(name, p.to(dtype).contiguous())
    return True


def _fold_state(sdfg, state):
    count = 0
    progressed = True
    while progressed:
        progressed = False
        for node in state.topological_compute_nodes():
            if not isinstance(node, donnx.ONNXOp):
                continue
            op = type(node).schema.name
            if op == "Split":
                if _fold_split(sdfg, state, node):
                    count += 1
                    progressed = True
                continue
            outs = state.out_edges(node)
            if len(outs) != 1 or not sdfg.arrays[outs[0].data.data].transient:
                continue
            out = outs[0].data.data
            if op == "Shape":
                value = torch.tensor(list(sdfg.arrays[P._in(state, node, "data")].shape), dtype=torch.int64)
            elif op in _EVAL:
                ins = {e.dst_conn: sdfg.constants.get(e.data.data) for e in state.in_edges(node)}
                if not ins or any(v is None for v in ins.values()):
                    continue
                with torch.no_grad():
                    value = _EVAL[op](node, {c: v for c, v in ins.items()})
            else:
                continue
            desc = sdfg.arrays[out]
            if tuple(value.shape) != tuple(desc.shape):
                raise ValueError("folding {} gave shape {}, the graph says {}".format(node, tuple(value.shape), desc.shape))
            state.remove_node(node)
            del sdfg.arrays[out]
            sdfg.add_constant(out, value.to(desc.dtype).contiguous())
            count += 1
            progressed = True
    return count


def fold_constants(sdfg):
    """Applies the folding to a fixpoint; returns the number of nodes replaced by constants."""
    n = sum(_fold_state(sdfg, st) for st in sdfg.states())
    if n:
        P.prune(sdfg)
    return n
