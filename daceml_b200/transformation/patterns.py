"""Fusion patterns over exported ONNX graphs; each is a function ``pattern(sdfg) -> number of rewrites``.

They recognise the sub-graphs the TorchScript / ONNX exporter emits at opset 12 (LayerNorm and GELU
decomposed, ``nn.Linear`` as ``Transpose -> MatMul -> Add`` or ``Gemm``, attention as MatMul / Mul /
Softmax / MatMul between head-split Reshape + Transpose pairs, Swish as ``Sigmoid -> Mul``, the
squeeze-excite branch of an MBConv block) and replace them by the fused operators that have one
kernel each.  A rewrite is only done when every intermediate array is a transient with no other
reader, so the visible results of the graph cannot change.
"""
import math

import torch

import daceml_b200.onnx as donnx
from daceml_b200 import sdfg as sd


# ---------------------------------------------------------------------------------------------
# graph helpers
# ---------------------------------------------------------------------------------------------
def _nodes(state, op):
    """The ``ONNX<op>`` nodes of the state; nodes removed by a rewrite during the walk are skipped."""
    cls = donnx.get_onnx_node(op)
    for n in [n for n in state.nodes() if type(n) is cls]:
        if n in state._nodes:
            yield n


def _in(state, node, conn):
    for e in state.in_edges_by_connector(node, conn):
        return e.data.data
    return None


def _out(state, node, conn=None):
    conn = conn or type(node).schema.outputs[0].name
    for e in state.out_edges_by_connector(node, conn):
        return e.data.data
    return None


def _producer(state, array):
    ws = [e.src for e in state.edges() if e.data.data == array and isinstance(e.src, donnx.ONNXOp)]
    return ws[0] if len(ws) == 1 else None


def _consumers(state, array):
    return [(e.dst, e.dst_conn) for e in state.edges() if e.data.data == array and isinstance(e.dst, donnx.ONNXOp)]


def _only_consumer(sdfg, state, array, op=None):
    """The single reader of a transient array (optionally required to be an ``ONNX<op>``)."""
    desc = sdfg.arrays.get(array)
    if desc is None or not desc.transient:
        return None, None
    cs = _consumers(state, array)
    if len(cs) != 1:
        return None, None
    node, conn = cs[0]
    if op is not None and type(node) is not donnx.get_onnx_node(op):
        return None, None
    return node, conn


def _const(sdfg, array):
    return sdfg.constants.get(array) if array is not None else None


def _scalar(sdfg, array):
    t = _const(sdfg, array)
    return float(t.reshape(-1)[0]) if t is not None and t.numel() == 1 else None


def _other_input(state, node, conn_a, conn_b, array):
    """For a commutative binary node fed by ``array``: the other operand's array."""
    a, b = _in(state, node, conn_a), _in(state, node, conn_b)
    if a == array:
        return b
    if b == array:
        return a
    return None


def _remove(state, nodes):
    for n in nodes:
        state.remove_node(n)


def _add_node(sdfg, state, op, label, inputs, outputs, **attrs):
    node = donnx.get_onnx_node(op)(label, **attrs)
    state.add_node(node)
    for conn, arr in inputs.items():
        if arr is not None:
            state.add_edge(state.add_read(arr), None, node, conn, sdfg.make_array_memlet(arr))
    for conn, arr in outputs.items():
        if arr is not None:
            state.add_edge(node, conn, state.add_write(arr), None, sdfg.make_array_memlet(arr))
    return node


def _attrs(node):
    return {k: getattr(node, k) for k in type(node).schema.attributes}


def prune(sdfg):
    """Drops access nodes without edges and transient arrays nothing refers to any more."""
    for state in sdfg.states():
        used = {e.src for e in state.edges()} | {e.dst for e in state.edges()}
        for n in state.nodes():
            if isinstance(n, sd.AccessNode) and n not in used:
                state.remove_node(n)
    referenced = {e.data.data for st in sdfg.states() for e in st.edges()}
    referenced |= {sdfg.root_of(n) for n in referenced} | {d.view_of for n, d in sdfg.arrays.items() if n in referenced and d.view_of}
    for name in [n for n, d in sdfg.arrays.items() if d.transient and n not in referenced]:
        del sdfg.arrays[name]
    for name in [n for n in sdfg.constants if n not in referenced]:
        del sdfg.constants[name]
        sdfg.arrays.pop(name, None)


def _each_state(fn):
    def pattern(sdfg):
        n = sum(fn(sdfg, st) for st in sdfg.states())
        if n:
            prune(sdfg)
        return n
    pattern.__name__ = fn.__name__
    pattern.__doc__ = fn.__doc__
    return pattern


# ---------------------------------------------------------------------------------------------
# element-wise chains
# ---------------------------------------------------------------------------------------------
@_each_state
def fuse_gelu(sdfg, state):
    """Div(x, sqrt 2) -> Erf -> Add(1) -> Mul(x, .) -> Mul(0.5)  =>  Gelu(x)."""
    count = 0
    for div in _nodes(state, "Div"):
        x = _in(state, div, "A")
        c = _scalar(sdfg, _in(state, div, "B"))
        if c is None or abs(c - math.sqrt(2.0)) > 1e-3:
            continue
        erf, _ = _only_consumer(sdfg, state, _out(state, div), "Erf")
        if erf is None:
            continue
        add, _ = _only_consumer(sdfg, state, _out(state, erf), "Add")
        if add is None or _scalar(sdfg, _other_input(state, add, "A", "B", _out(state, erf))) != 1.0:
            continue
        mul1, _ = _only_consumer(sdfg, state, _out(state, add), "Mul")
        if mul1 is None or _other_input(state, mul1, "A", "B", _out(state, add)) != x:
            continue
        mul2, _ = _only_consumer(sdfg, state, _out(state, mul1), "Mul")
        if mul2 is None or _scalar(sdfg, _other_input(state, mul2, "A", "B", _out(state, mul1))) != 0.5:
            continue
        y = _out(state, mul2)
        _remove(state, [div, erf, add, mul1, mul2])
        _add_node(sdfg, state, "Gelu", div.label + "_gelu", dict(X=x), dict(Y=y))
        count += 1
    return count


@_each_state
def fuse_swish(sdfg, state):
    """Sigmoid(x) -> Mul(x, .)  =>  Swish(x)."""
    count = 0
    for sig in _nodes(state, "Sigmoid"):
        x = _in(state, sig, "X")
        mul, _ = _only_consumer(sdfg, state, _out(state, sig), "Mul")
        if mul is None or _other_input(state, mul, "A", "B", _out(state, sig)) != x:
            continue
        y = _out(state, mul)
        _remove(state, [sig, mul])
        _add_node(sdfg, state, "Swish", sig.label + "_swish", dict(X=x), dict(Y=y))
        count += 1
    return count


@_each_state
def fuse_layernorm(sdfg, state):
    """ReduceMean -> Sub [-> Cast] -> Pow(2) -> ReduceMean -> Add(eps) -> Sqrt -> Div [-> Cast] -> Mul(gamma) -> Add(beta)
    =>  LayerNormalization (statistics in fp32 whatever the storage type)."""
    count = 0
    for mean in _nodes(state, "ReduceMean"):
        x = _in(state, mean, "data")
        rank = len(sdfg.arrays[x].shape)
        if mean.axes is None or [a % rank for a in mean.axes] != [rank - 1]:
            continue
        sub, conn = _only_consumer(sdfg, state, _out(state, mean), "Sub")
        if sub is None or conn != "B" or _in(state, sub, "A") != x:
            continue
        d = _out(state, sub)
        # half-precision exports widen the centred values for the variance: Sub -> Cast(wide) ... Div -> Cast(back)
        cast_up, _ = _only_consumer(sdfg, state, d, "Cast")
        if cast_up is not None:
            d = _out(state, cast_up)
        users = _consumers(state, d)
        if len(users) != 2 or not sdfg.arrays[d].transient:
            continue
        pw = next((n for n, _ in users if type(n) is donnx.ONNXPow), None)
        dv = next((n for n, c in users if type(n) is donnx.ONNXDiv and c == "A"), None)
        if pw is None or dv is None or _scalar(sdfg, _in(state, pw, "Y")) != 2.0:
            continue
        var, _ = _only_consumer(sdfg, state, _out(state, pw), "ReduceMean")
        if var is None or var.axes is None or [a % rank for a in var.axes] != [rank - 1]:
            continue
        add, _ = _only_consumer(sdfg, state, _out(state, var), "Add")
        eps = _scalar(sdfg, _other_input(state, add, "A", "B", _out(state, var))) if add is not None else None
        if eps is None:
            continue
        sq, _ = _only_consumer(sdfg, state, _out(state, add), "Sqrt")
        if sq is None or _only_consumer(sdfg, state, _out(state, sq), "Div")[0] is not dv:
            continue
        chain, y, gamma, beta = [mean, sub, pw, var, add, sq, dv], _out(state, dv), None, None
        if cast_up is not None:
            cast_dn, _ = _only_consumer(sdfg, state, y, "Cast")
            if cast_dn is None or sdfg.arrays[_out(state, cast_dn)].dtype != sdfg.arrays[x].dtype:
                continue
            chain += [cast_up, cast_dn]
            y = _out(state, cast_dn)
        mul, _ = _only_consumer(sdfg, state, y, "Mul")
        if mul is not None:
            g = _other_input(state, mul, "A", "B", y)
            if _const(sdfg, g) is not None and _const(sdfg, g).dim() == 1:
                gamma, y = g, _out(state, mul)
                chain.append(mul)
                addb, _ = _only_consumer(sdfg, state, y, "Add")
                if addb is not None:
                    b = _other_input(state, addb, "A", "B", y)
                    if _const(sdfg, b) is not None and _const(sdfg, b).dim() == 1:
                        beta, y = b, _out(state, addb)
                        chain.append(addb)
        _remove(state, chain)
        _add_node(sdfg, state, "LayerNormalization", mean.label + "_layernorm", dict(X=x, Scale=gamma, B=beta), dict(Y=y),
                  axis=-1, epsilon=eps)
        count += 1
    return count


# ---------------------------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------------------------
@_each_state
def fuse_linear(sdfg, state):
    """Transpose(W) -> MatMul -> Add(bias), MatMul(x, W^T constant) -> Add(bias), MatMul alone and Gemm  =>  FusedMatMul."""
    count = 0
    for mm in _nodes(state, "MatMul"):
        a, b = _in(state, mm, "A"), _in(state, mm, "B")
        if len(sdfg.arrays[b].shape) != 2:
            continue
        remove, weight, trans_b = [mm], b, 0
        tr = _producer(state, b)
        if (tr is not None and type(tr) is donnx.ONNXTranspose and list(tr.perm or [1, 0]) == [1, 0]
                and _only_consumer(sdfg, state, b)[0] is mm and _const(sdfg, _in(state, tr, "data")) is not None):
            weight, trans_b = _in(state, tr, "data"), 1
            remove.append(tr)
        elif _const(sdfg, b) is not None:
            # a weight stored [in, out] (the exporter folded its Transpose): keep a [out, in] copy, the K-major
            # operand layout of the fast matrix-product kernels
            weight, trans_b = b + "_T", 1
            if weight not in sdfg.constants:
                sdfg.add_constant(weight, _const(sdfg, b).t().contiguous())
        y, bias = _out(state, mm), None
        add, _ = _only_consumer(sdfg, state, y, "Add")
        if add is not None:
            cand = _other_input(state, add, "A", "B", y)
            ct = _const(sdfg, cand)
            if ct is not None and ct.dim() == 1 and ct.shape[0] == sdfg.arrays[y].shape[-1]:
                bias, y = cand, _out(state, add)
                remove.append(add)
        _remove(state, remove)
        _add_node(sdfg, state, "FusedMatMul", mm.label + "_fused", dict(A=a, B=weight, Bias=bias), dict(Y=y), transB=trans_b)
        count += 1
    for gm in _nodes(state, "Gemm"):
        c = _in(state, gm, "C")
        if int(gm.transA) != 0 or (c is not None and (float(gm.beta) != 1.0 or len(sdfg.arrays[c].shape) != 1)):
            continue
        a, b, y = _in(state, gm, "A"), _in(state, gm, "B"), _out(state, gm)
        _remove(state, [gm])
        _add_node(sdfg, state, "FusedMatMul", gm.label + "_fused", dict(A=a, B=b, Bias=c), dict(Y=y), transB=int(gm.transB),
                  alpha=float(gm.alpha))
        count += 1
    return count


def _rebuild_fused(sdfg, state, node, **changes):
    """Replaces a FusedMatMul by a copy with some connectors / attributes changed."""
    ins = {p.name: _in(state, node, p.name) for p in type(node).schema.inputs}
    outs = dict(Y=_out(state, node))
    attrs = _attrs(node)
    for k, v in changes.items():
        if k in attrs:
            attrs[k] = v
        elif k == "Y":
            outs["Y"] = v
        else:
            ins[k] = v
    _remove(state, [node])
    return _add_node(sdfg, state, "FusedMatMul", node.label, ins, outs, **attrs)


@_each_state
def fuse_matmul_epilogue(sdfg, state):
    """FusedMatMul -> Relu | Gelu | Swish, -> Add(residual), -> LayerNormalization  =>  one FusedMatMul."""
    count = 0
    for fm in _nodes(state, "FusedMatMul"):
        y = _out(state, fm)
        nxt, conn = _only_consumer(sdfg, state, y)
        if nxt is None:
            continue
        has_res, has_ln = _in(state, fm, "Residual") is not None, fm.ln_epsilon is not None
        kind = type(nxt).schema.name
        if kind in ("Relu", "Gelu", "Swish") and not fm.activation and not has_res and not has_ln:
            out = _out(state, nxt)
            _remove(state, [nxt])
            _rebuild_fused(sdfg, state, fm, activation=kind, Y=out)
            count += 1
        elif kind == "Add" and not has_res and not has_ln:
            other = _other_input(state, nxt, "A", "B", y)
            if other is None or tuple(sdfg.arrays[other].shape) != tuple(sdfg.arrays[y].shape):
                continue
            out = _out(state, nxt)
            _remove(state, [nxt])
            _rebuild_fused(sdfg, state, fm, Residual=other, Y=out)
            count += 1
        elif kind == "LayerNormalization" and not has_ln and conn == "X" and _in(state, nxt, "Residual") is None:
            rank = len(sdfg.arrays[y].shape)
            if int(nxt.axis) % rank != rank - 1:
                continue
            out = _out(state, nxt)
            scale, shift = _in(state, nxt, "Scale"), _in(state, nxt, "B")
            _remove(state, [nxt])
            _rebuild_fused(sdfg, state, fm, LnScale=scale, LnBias=shift, ln_epsilon=float(nxt.epsilon), Y=out)
            count += 1
    return count


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------
def _head_split(sdfg, state, array, perm):
    """``array`` = Transpose(perm)(Reshape[B,S,h,d](src)) with single-use intermediates: returns (src, [nodes], h, d)."""
    tr = _producer(state, array)
    if tr is None or type(tr) is not donnx.ONNXTranspose or list(tr.perm or []) != list(perm):
        return None
    if _only_consumer(sdfg, state, array)[0] is None:
        return None
    mid = _in(state, tr, "data")
    rs = _producer(state, mid)
    if rs is None or type(rs) is not donnx.ONNXReshape or _only_consumer(sdfg, state, mid)[0] is not tr:
        return None
    src = _in(state, rs, "data")
    shp, sshp = sdfg.arrays[mid].shape, sdfg.arrays[src].shape
    if len(shp) != 4 or len(sshp) != 3 or sshp[2] != shp[2] * shp[3]:
        return None
    return src, [tr, rs], shp[2], shp[3]


@_each_state
def fuse_attention(sdfg, state):
    """MatMul(Q, K^T) -> Mul(scale) [-> Add(mask)] -> Softmax(last axis) -> MatMul(., V) -> Transpose -> Reshape, with the
    head-split Reshape / Transpose pairs in front  =>  Attention(Q, K, V[, Mask]) on [B, S, H] tensors."""
    count = 0
    for sm in _nodes(state, "Softmax"):
        scores = _in(state, sm, "input")
        rank = len(sdfg.arrays[scores].shape)
        if rank != 4 or int(sm.axis) % rank != 3:
            continue
        chain, mask = [sm], None
        prev = _producer(state, scores)
        if prev is not None and type(prev) is donnx.ONNXAdd and _only_consumer(sdfg, state, scores)[0] is sm:
            # additive mask: a [B, S_kv] constant of the scores' type reshaped to [B, 1, 1, S_kv] (the layout the kernel
            # reads); a [1, S] row broadcast over the batch, an [S, S] causal or relative-bias constant and anything
            # else stay an Add in front of the Softmax
            a, b = _in(state, prev, "A"), _in(state, prev, "B")
            shp = sdfg.arrays[scores].shape
            cand = [t for t in (a, b) if _producer(state, t) is not None and type(_producer(state, t)) is donnx.ONNXReshape
                    and _const(sdfg, _in(state, _producer(state, t), "data")) is not None]
            if len(cand) == 1:
                rs = _producer(state, cand[0])
                mask = _in(state, rs, "data")
                const = _const(sdfg, mask)
                if (tuple(const.shape) != (shp[0], shp[3]) or const.dtype != sdfg.arrays[scores].dtype
                        or tuple(sdfg.arrays[cand[0]].shape) != (shp[0], 1, 1, shp[3])):
                    continue
                chain += [prev]
                if _only_consumer(sdfg, state, cand[0])[0] is prev:
                    chain += [rs]  # a Reshape that other layers read as well stays; prune() drops it once unused
            else:
                # a mask computed at run time (or fed in): any [B, 1, 1, S] operand of the scores' type
                cand = [t for t in (a, b) if tuple(sdfg.arrays[t].shape) == (shp[0], 1, 1, shp[3])
                        and sdfg.arrays[t].dtype == sdfg.arrays[scores].dtype]
                if len(cand) != 1:
                    continue
                mask = cand[0]
                chain += [prev]
            scores = a if cand[0] == b else b
            prev = _producer(state, scores)
        if prev is None or type(prev) is not donnx.ONNXMul or _only_consumer(sdfg, state, scores)[0] is None:
            continue
        raw = _in(state, prev, "A") if _scalar(sdfg, _in(state, prev, "B")) is not None else _in(state, prev, "B")
        scale = _scalar(sdfg, _other_input(state, prev, "A", "B", raw))
        qk = _producer(state, raw)
        if scale is None or qk is None or type(qk) is not donnx.ONNXMatMul or _only_consumer(sdfg, state, raw)[0] is not prev:
            continue
        chain += [prev, qk]
        q = _head_split(sdfg, state, _in(state, qk, "A"), (0, 2, 1, 3))
        k = _head_split(sdfg, state, _in(state, qk, "B"), (0, 2, 3, 1))
        pv, conn = _only_consumer(sdfg, state, _out(state, sm), "MatMul")
        if q is None or k is None or pv is None or conn != "A":
            continue
        v = _head_split(sdfg, state, _in(state, pv, "B"), (0, 2, 1, 3))
        tr, _ = _only_consumer(sdfg, state, _out(state, pv), "Transpose")
        if v is None or tr is None or list(tr.perm or []) != [0, 2, 1, 3]:
            continue
        rs2, _ = _only_consumer(sdfg, state, _out(state, tr), "Reshape")
        if rs2 is None or (q[2], q[3]) != (k[2], k[3]) or (q[2], q[3]) != (v[2], v[3]):
            continue
        if mask is not None and int(math.prod(sdfg.arrays[mask].shape)) != sdfg.arrays[q[0]].shape[0] * sdfg.arrays[k[0]].shape[1]:
            continue
        # the fused kernel is fp16 with 64-wide heads; anything else stays MatMul / Softmax / MatMul
        if sdfg.arrays[q[0]].dtype != torch.float16 or q[3] != 64:
            continue
        out = _out(state, rs2)
        _remove(state, chain + [pv, tr, rs2] + q[1] + k[1] + v[1])
        _add_node(sdfg, state, "Attention", sm.label + "_attention", dict(Q=q[0], K=k[0], V=v[0], Mask=mask), dict(Y=out),
                  num_heads=q[2], scale=scale)
        count += 1
    return count


@_each_state
def pack_qkv(sdfg, state):
    """Three FusedMatMul(x, W_q|k|v) feeding one Attention  =>  one FusedMatMul with the weights concatenated and the
    Attention reading the packed [B, S, 3H] result."""
    count = 0
    for att in _nodes(state, "Attention"):
        arrays = [_in(state, att, c) for c in ("Q", "K", "V")]
        if any(a is None for a in arrays):
            continue
        prods = [_producer(state, a) for a in arrays]
        if any(p is None or type(p) is not donnx.ONNXFusedMatMul for p in prods) or len({id(p) for p in prods}) != 3:
            continue
        if any(_only_consumer(sdfg, state, a)[0] is not att for a in arrays):
            continue
        if any(p.activation or p.ln_epsilon is not None or _in(state, p, "Residual") is not None or int(p.transB) != 1
               or float(p.alpha) != 1.0 for p in prods):
            continue
        src = {_in(state, p, "A") for p in prods}
        ws = [_const(sdfg, _in(state, p, "B")) for p in prods]
        bs = [_const(sdfg, _in(state, p, "Bias")) for p in prods]
        if len(src) != 1 or any(w is None for w in ws) or len({tuple(w.shape) for w in ws}) != 1:
            continue
        if any(b is None for b in bs) and not all(b is None for b in bs):
            continue
        x = src.pop()
        wname = att.label + "_wqkv"
        sdfg.add_constant(wname, torch.cat(ws, 0).contiguous())
        bname = None
        if bs[0] is not None:
            bname = att.label + "_bqkv"
            sdfg.add_constant(bname, torch.cat(bs, 0).contiguous())
        shp = sdfg.arrays[arrays[0]].shape
        packed = att.label + "_qkv"
        sdfg.add_transient(packed, tuple(shp[:-1]) + (3 * shp[-1], ), sdfg.arrays[arrays[0]].dtype)
        mask, out, attrs = _in(state, att, "Mask"), _out(state, att), _attrs(att)
        _remove(state, prods + [att])
        _add_node(sdfg, state, "FusedMatMul", att.label + "_qkv_proj", dict(A=x, B=wname, Bias=bname), dict(Y=packed), transB=1)
        _add_node(sdfg, state, "Attention", att.label, dict(Q=packed, Mask=mask), dict(Y=out), **attrs)
        count += 1
    return count


# ---------------------------------------------------------------------------------------------
# convolution blocks
# ---------------------------------------------------------------------------------------------
def batchnorm_affine(sdfg, state, bn):
    """Inference BatchNormalization as a per-channel ``a * x + b`` (fp32 on the host); None unless the four statistics
    tensors are constants."""
    ts = [_const(sdfg, _in(state, bn, c)) for c in ("scale", "B", "mean", "var")]
    if any(t is None for t in ts):
        return None
    scale, shift, mean, var = (t.detach().float().cpu() for t in ts)
    a = scale / torch.sqrt(var + float(bn.epsilon))
    return a, shift - mean * a


@_each_state
def fold_batchnorm_into_conv(sdfg, state):
    """Conv(W, b) -> BatchNormalization(constants)  =>  Conv(a * W, a * b + shift): the exporter does this itself for
    modules in eval mode; graphs from elsewhere may still carry the pair."""
    count = 0
    for bn in _nodes(state, "BatchNormalization"):
        x = _in(state, bn, "X")
        conv = _producer(state, x)
        if conv is None or type(conv) is not donnx.ONNXConv or _only_consumer(sdfg, state, x)[0] is not bn:
            continue
        w, b = _const(sdfg, _in(state, conv, "W")), _in(state, conv, "B")
        ab = batchnorm_affine(sdfg, state, bn)
        if w is None or ab is None or (b is not None and _const(sdfg, b) is None):
            continue
        a, shift = ab
        dtype, dev = w.dtype, w.device
        wn, bnm = bn.label + "_w", bn.label + "_b"
        sdfg.add_constant(wn, (w.float().cpu() * a.reshape(-1, 1, 1, 1)).to(dtype).to(dev).contiguous())
        bias = _const(sdfg, b).float().cpu() if b is not None else torch.zeros_like(a)
        sdfg.add_constant(bnm, (bias * a + shift).to(dtype).to(dev).contiguous())
        ins, y, attrs = dict(X=_in(state, conv, "X"), W=wn, B=bnm), _out(state, bn), _attrs(conv)
        _remove(state, [conv, bn])
        _add_node(sdfg, state, "Conv", conv.label, ins, dict(Y=y), **attrs)
        count += 1
    return count


@_each_state
def fuse_conv(sdfg, state):
    """Conv -> Swish | Relu  =>  FusedConv(activation); a Conv left alone also becomes a FusedConv so that the gate,
    residual and pooling patterns below can attach to it."""
    count = 0
    for cv in _nodes(state, "Conv"):
        if getattr(cv, "auto_pad", "NOTSET") not in ("NOTSET", "VALID"):
            continue
        y = _out(state, cv)
        act = ""
        nxt, _ = _only_consumer(sdfg, state, y)
        drop = [cv]
        if nxt is not None and type(nxt).schema.name in ("Swish", "Relu"):
            act, y = type(nxt).schema.name, _out(state, nxt)
            drop.append(nxt)
        ins = dict(X=_in(state, cv, "X"), W=_in(state, cv, "W"), B=_in(state, cv, "B"))
        attrs = dict(dilations=cv.dilations, group=cv.group, kernel_shape=cv.kernel_shape, pads=cv.pads, strides=cv.strides)
        _remove(state, drop)
        _add_node(sdfg, state, "FusedConv", cv.label + "_fused", ins, dict(Y=y), activation=act, **attrs)
        count += 1
    return count


def _rebuild_conv(sdfg, state, node, **changes):
    ins = {p.name: _in(state, node, p.name) for p in type(node).schema.inputs}
    outs = dict(Y=_out(state, node, "Y"), Pool=_out(state, node, "Pool"))
    attrs = _attrs(node)
    for k, v in changes.items():
        if k in attrs:
            attrs[k] = v
        elif k in outs:
            outs[k] = v
        else:
            ins[k] = v
    _remove(state, [node])
    return _add_node(sdfg, state, "FusedConv", node.label, ins, outs, **attrs)


@_each_state
def fuse_squeeze_excite(sdfg, state):
    """GlobalAveragePool -> FusedConv(1x1, Swish) -> FusedConv(1x1) -> Sigmoid -> Mul(gate, y) -> FusedConv(1x1)
    =>  pooling folded into the producer of y, one SqueezeExcite launch, the gate applied on the consumer's input."""
    count = 0
    for gap in _nodes(state, "GlobalAveragePool"):
        y = _in(state, gap, "X")
        c1, _ = _only_consumer(sdfg, state, _out(state, gap), "FusedConv")
        if c1 is None or c1.activation != "Swish":
            continue
        c2, _ = _only_consumer(sdfg, state, _out(state, c1, "Y"), "FusedConv")
        if c2 is None or c2.activation:
            continue
        sig, _ = _only_consumer(sdfg, state, _out(state, c2, "Y"), "Sigmoid")
        if sig is None:
            continue
        gate = _out(state, sig)
        mul, _ = _only_consumer(sdfg, state, gate, "Mul")
        if mul is None or _other_input(state, mul, "A", "B", gate) != y:
            continue
        w1, w2 = _const(sdfg, _in(state, c1, "W")), _const(sdfg, _in(state, c2, "W"))
        if w1 is None or w2 is None or tuple(w1.shape[2:]) != (1, 1) or tuple(w2.shape[2:]) != (1, 1):
            continue
        if any(int(c.group or 1) != 1 or _in(state, c, "Gate") is not None or _in(state, c, "Residual") is not None
               for c in (c1, c2)):
            continue
        gated = _out(state, mul)
        cons, conn = _only_consumer(sdfg, state, gated, "FusedConv")
        prod = _producer(state, y)
        users_y = _consumers(state, y)
        if (cons is None or conn != "X" or _in(state, cons, "Gate") is not None or prod is None
                or type(prod) is not donnx.ONNXFusedConv or len(users_y) != 2):
            continue
        w1n, w2n = gap.label + "_se_w1", gap.label + "_se_w2"
        sdfg.add_constant(w1n, w1.reshape(w1.shape[0], w1.shape[1]).contiguous())
        sdfg.add_constant(w2n, w2.reshape(w2.shape[0], w2.shape[1]).contiguous())
        b1, b2 = _in(state, c1, "B"), _in(state, c2, "B")
        pooled = _out(state, gap)
        _remove(state, [gap, c1, c2, sig, mul])
        _rebuild_conv(sdfg, state, prod, Pool=pooled)
        _add_node(sdfg, state, "SqueezeExcite", gap.label + "_se", dict(X=pooled, W1=w1n, B1=b1, W2=w2n, B2=b2), dict(Y=gate))
        _rebuild_conv(sdfg, state, cons, X=y, Gate=gate)
        count += 1
    return count


@_each_state
def fuse_conv_residual(sdfg, state):
    """FusedConv -> Add(residual)  =>  FusedConv with a Residual input."""
    count = 0
    for cv in _nodes(state, "FusedConv"):
        if _in(state, cv, "Residual") is not None or _out(state, cv, "Pool") is not None:
            continue
        y = _out(state, cv, "Y")
        add, _ = _only_consumer(sdfg, state, y, "Add")
        if add is None:
            continue
        other = _other_input(state, add, "A", "B", y)
        if other is None or tuple(sdfg.arrays[other].shape) != tuple(sdfg.arrays[y].shape):
            continue
        out = _out(state, add)
        _remove(state, [add])
        _rebuild_conv(sdfg, state, cv, Residual=other, Y=out)
        count += 1
    return count


@_each_state
def remove_identity(sdfg, state):
    """producer -> t -> Identity -> y  =>  producer -> y, when t is a transient nobody else reads."""
    count = 0
    for ident in _nodes(state, "Identity"):
        t, y = _in(state, ident, "input"), _out(state, ident)
        prod = _producer(state, t)
        if prod is None or _only_consumer(sdfg, state, t)[0] is not ident:
            continue
        if sdfg.arrays[t].shape != sdfg.arrays[y].shape or sdfg.arrays[t].dtype != sdfg.arrays[y].dtype:
            continue
        edge = next(e for e in state.out_edges(prod) if e.data.data == t)
        conn = edge.src_conn
        state.remove_edge(edge)
        _remove(state, [ident])
        state.add_edge(prod, conn, state.add_write(y), None, sdfg.make_array_memlet(y))
        count += 1
    return count


@_each_state
def alias_reshapes(sdfg, state):
    """Reshape / Flatten / Squeeze / Unsqueeze / Identity into a transient  =>  no launch: the output becomes a view of
    the input's storage (all arrays are contiguous, and an exported graph writes every array once); when the output is
    a result of the model, the input becomes a view of it instead, so that its producer writes the result in place.
    Run after the fusion patterns, which look for these nodes."""
    count = 0
    for op, i, o in (("Reshape", "data", "reshaped"), ("Flatten", "input", "output"), ("Squeeze", "data", "squeezed"),
                     ("Unsqueeze", "data", "expanded"), ("Identity", "input", "output")):
        for node in _nodes(state, op):
            src, dst = _in(state, node, i), _out(state, node, o)
            a, b = sdfg.arrays[src], sdfg.arrays[dst]
            if a.dtype != b.dtype or a.total_size() != b.total_size() or src in sdfg.constants:
                continue
            if len([e for e in state.edges() if e.data.data == dst and isinstance(e.src, donnx.ONNXOp)]) != 1:
                continue
            if b.transient:
                _remove(state, [node])
                b.view_of = src
            else:
                # the reshape feeds a model output: the producer of its input writes straight into the output's storage,
                # provided nothing else reads that storage (under any of the names that view it)
                root = sdfg.root_of(src)
                r = sdfg.arrays[root]
                readers = [e.dst for e in state.edges() if isinstance(e.dst, donnx.ONNXOp) and sdfg.root_of(e.data.data) == root]
                if not r.transient or root in sdfg.constants or _producer(state, root) is None or readers != [node]:
                    continue
                _remove(state, [node])
                r.view_of = dst
            count += 1
    return count


PATTERNS = [remove_identity, fold_batchnorm_into_conv, fuse_gelu, fuse_swish, fuse_layernorm, fuse_linear, fuse_matmul_epilogue, fuse_attention, pack_qkv, fuse_conv,
            fuse_squeeze_excite, fuse_conv_residual]
