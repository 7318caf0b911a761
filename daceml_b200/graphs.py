"""SDFG builders for the graphs the ONNX exporter produces for the benchmark configurations.

The reference obtains these graphs with ``torch.onnx.export(..., opset_version=12)`` followed by
``ONNXModel`` (``daceml/torch/module.py:269-315``, ``daceml/onnx/onnx_importer.py:197-338``).
Neither ``onnx`` nor DaCe is available to this build, so the same node lists (recorded from the
TorchScript exporter at opset 12) are written down here as builders.  Every builder has two
forms: ``fused=False`` is the exported node-for-node graph (LayerNorm and GELU decomposed,
weights as ``Transpose -> MatMul -> Add``), ``fused=True`` is the graph after the fusion pass.
Weights are bound as SDFG constants, like the importer's ``weights`` dictionary
(``onnx_importer.py:190-193``).
"""
import itertools
import math

import torch

import daceml_b200.onnx as donnx
from daceml_b200 import sdfg as sd


class GraphBuilder:
    """Adds library nodes to one state and names their transient outputs."""

    def __init__(self, name, dtype):
        self.sdfg = sd.SDFG(name)
        self.state = self.sdfg.add_state()
        self.dtype = dtype
        self._ids = itertools.count()

    def input(self, name, shape, dtype=None):
        self.sdfg.add_array(name, shape, dtype or self.dtype)
        return name

    def output(self, name, shape, dtype=None):
        self.sdfg.add_array(name, shape, dtype or self.dtype)
        return name

    def constant(self, name, tensor):
        self.sdfg.add_constant(name, tensor.detach().contiguous())
        return name

    def scalar(self, value, name=None):
        name = name or "c{}".format(next(self._ids))
        return self.constant(name, torch.tensor(value, dtype=self.dtype))

    def shape(self, name):
        return self.sdfg.arrays[name].shape

    def node(self, op, inputs, out_shape, out=None, out_conn=None, out_dtype=None, **attrs):
        """Adds ``ONNX<op>`` reading ``inputs`` (connector -> array) and writing a new transient
        (or the array ``out``); returns the output array's name."""
        cls = donnx.get_onnx_node(op)
        idx = next(self._ids)
        node = cls("{}_{}".format(op, idx), **attrs)
        self.state.add_node(node)
        for conn, arr in inputs.items():
            if arr is None:
                continue
            self.state.add_edge(self.state.add_read(arr), None, node, conn, self.sdfg.make_array_memlet(arr))
        if out is None:
            out = "t{}_{}".format(idx, op.lower())
            self.sdfg.add_transient(out, out_shape, out_dtype or self.dtype)
        conn = out_conn or cls.schema.outputs[0].name
        self.state.add_edge(node, conn, self.state.add_write(out), None, self.sdfg.make_array_memlet(out))
        return out

    def extra_output(self, producer_array, op_conn, shape, dtype=None, name=None):
        """Connects a further output connector of the node that wrote ``producer_array``."""
        node = next(e.src for e in self.state.edges() if e.data.data == producer_array and not isinstance(e.src, sd.AccessNode))
        name = name or "t{}_{}".format(next(self._ids), op_conn.lower())
        self.sdfg.add_transient(name, shape, dtype or self.dtype)
        self.state.add_edge(node, op_conn, self.state.add_write(name), None, self.sdfg.make_array_memlet(name))
        return name


# ---------------------------------------------------------------------------------------------
# config 2: MLP  (Gemm(transB=1) -> Relu -> Gemm -> Relu -> Gemm -> LogSoftmax(axis=1))
# ---------------------------------------------------------------------------------------------
def mlp_sdfg(params, batch, fused=True, dtype=torch.float32):
    g = GraphBuilder("mlp", dtype)
    x = g.input("input", (batch, params["w1"].shape[1]))
    h = x
    for i in (1, 2, 3):
        w, b = params["w%d" % i], params["b%d" % i]
        wn, bn = g.constant("fc%d_weight" % i, w), g.constant("fc%d_bias" % i, b)
        shape = (batch, w.shape[0])
        if fused:
            h = g.node("FusedMatMul", dict(A=h, B=wn, Bias=bn), shape, transB=1, activation="Relu" if i < 3 else "")
        else:
            h = g.node("Gemm", dict(A=h, B=wn, C=bn), shape, alpha=1.0, beta=1.0, transB=1)
            if i < 3:
                h = g.node("Relu", dict(X=h), shape)
    out = g.output("__return", g.shape(h))
    g.node("LogSoftmax", dict(input=h), g.shape(h), out=out, axis=1)
    return g.sdfg


# ---------------------------------------------------------------------------------------------
# configs 3 / 5: post-LN BERT encoder layer
# ---------------------------------------------------------------------------------------------
def _layernorm_chain(g, x, gamma, beta, eps, shape):
    red = tuple(shape[:-1]) + (1, )
    mean = g.node("ReduceMean", dict(data=x), red, axes=[-1], keepdims=1)
    d = g.node("Sub", dict(A=x, B=mean), shape)
    sq = g.node("Pow", dict(X=d, Y=g.scalar(2.0)), shape)
    var = g.node("ReduceMean", dict(data=sq), red, axes=[-1], keepdims=1)
    ve = g.node("Add", dict(A=var, B=g.scalar(eps)), red)
    std = g.node("Sqrt", dict(X=ve), red)
    nrm = g.node("Div", dict(A=d, B=std), shape)
    sc = g.node("Mul", dict(A=nrm, B=gamma), shape)
    return g.node("Add", dict(A=sc, B=beta), shape)


def _gelu_chain(g, x, shape):
    d = g.node("Div", dict(A=x, B=g.scalar(1.41421354)), shape)
    e = g.node("Erf", dict(input=d), shape)
    a = g.node("Add", dict(A=e, B=g.scalar(1.0)), shape)
    m = g.node("Mul", dict(A=x, B=a), shape)
    return g.node("Mul", dict(A=m, B=g.scalar(0.5)), shape)


def bert_layer_sdfg(p, batch, seq, heads, fused=True, eps=1e-12, dtype=torch.float16, name="bert_layer",
                    out_name="__return", fuse_layernorm=True):
    """``p`` holds ``wq, bq, wk, bk, wv, bv, wo, bo, ln1_g, ln1_b, w1, b1, w2, b2, ln2_g, ln2_b`` with
    nn.Linear ``[out, in]`` weight layout (and optionally ``mask`` of shape [batch, seq])."""
    hidden = p["wq"].shape[0]
    ffn = p["w1"].shape[0]
    d = hidden // heads
    g = GraphBuilder(name, dtype)
    x = g.input("input", (batch, seq, hidden))
    c = {k: g.constant(k, v.to(dtype)) for k, v in p.items() if k != "mask" and v is not None}
    mask = g.constant("mask", p["mask"].to(dtype)) if p.get("mask") is not None else None
    bsh = (batch, seq, hidden)
    if fused:
        wqkv = g.constant("wqkv", torch.cat([p["wq"], p["wk"], p["wv"]], 0).to(dtype))
        bqkv = g.constant("bqkv", torch.cat([p["bq"], p["bk"], p["bv"]], 0).to(dtype))
        qkv = g.node("FusedMatMul", dict(A=x, B=wqkv, Bias=bqkv), (batch, seq, 3 * hidden), transB=1)
        ctx = g.node("Attention", dict(Q=qkv, Mask=mask), bsh, num_heads=heads, scale=1.0 / math.sqrt(d))
        y = g.output(out_name, bsh)
        if fuse_layernorm:  # the residual Add and the LayerNorm chain ride in the epilogue of the matrix product
            h1 = g.node("FusedMatMul", dict(A=ctx, B=c["wo"], Bias=c["bo"], Residual=x, LnScale=c["ln1_g"], LnBias=c["ln1_b"]),
                        bsh, transB=1, ln_epsilon=eps)
        else:
            attn = g.node("FusedMatMul", dict(A=ctx, B=c["wo"], Bias=c["bo"], Residual=x), bsh, transB=1)
            h1 = g.node("LayerNormalization", dict(X=attn, Scale=c["ln1_g"], B=c["ln1_b"]), bsh, axis=-1, epsilon=eps)
        inter = g.node("FusedMatMul", dict(A=h1, B=c["w1"], Bias=c["b1"]), (batch, seq, ffn), transB=1,
                       activation="Gelu")
        if fuse_layernorm:
            g.node("FusedMatMul", dict(A=inter, B=c["w2"], Bias=c["b2"], Residual=h1, LnScale=c["ln2_g"], LnBias=c["ln2_b"]),
                   bsh, out=y, transB=1, ln_epsilon=eps)
        else:
            out = g.node("FusedMatMul", dict(A=inter, B=c["w2"], Bias=c["b2"], Residual=h1), bsh, transB=1)
            g.node("LayerNormalization", dict(X=out, Scale=c["ln2_g"], B=c["ln2_b"]), bsh, out=y, axis=-1, epsilon=eps)
        return g.sdfg

    def linear(inp, w, b, n_out):
        wt = g.node("Transpose", dict(data=w), tuple(reversed(g.shape(w))), perm=[1, 0])
        mm = g.node("MatMul", dict(A=inp, B=wt), (batch, seq, n_out))
        return g.node("Add", dict(A=mm, B=b), (batch, seq, n_out))

    def split_heads(t, perm):
        r = g.node("Reshape", dict(data=t), (batch, seq, heads, d))
        shape = tuple((batch, seq, heads, d)[i] for i in perm)
        return g.node("Transpose", dict(data=r), shape, perm=list(perm))

    q = split_heads(linear(x, c["wq"], c["bq"], hidden), (0, 2, 1, 3))
    k = split_heads(linear(x, c["wk"], c["bk"], hidden), (0, 2, 3, 1))
    v = split_heads(linear(x, c["wv"], c["bv"], hidden), (0, 2, 1, 3))
    scores = g.node("MatMul", dict(A=q, B=k), (batch, heads, seq, seq))
    scores = g.node("Mul", dict(A=scores, B=g.scalar(1.0 / math.sqrt(d))), (batch, heads, seq, seq))
    if mask is not None:
        m4 = g.node("Reshape", dict(data=mask), (batch, 1, 1, seq))
        scores = g.node("Add", dict(A=scores, B=m4), (batch, heads, seq, seq))
    probs = g.node("Softmax", dict(input=scores), (batch, heads, seq, seq), axis=3)
    ctx = g.node("MatMul", dict(A=probs, B=v), (batch, heads, seq, d))
    ctx = g.node("Transpose", dict(data=ctx), (batch, seq, heads, d), perm=[0, 2, 1, 3])
    ctx = g.node("Reshape", dict(data=ctx), bsh)
    attn = g.node("Add", dict(A=linear(ctx, c["wo"], c["bo"], hidden), B=x), bsh)
    h1 = _layernorm_chain(g, attn, c["ln1_g"], c["ln1_b"], eps, bsh)
    inter = _gelu_chain(g, linear(h1, c["w1"], c["b1"], ffn), (batch, seq, ffn))
    out = g.node("Add", dict(A=linear(inter, c["w2"], c["b2"], hidden), B=h1), bsh)
    ln = _layernorm_chain(g, out, c["ln2_g"], c["ln2_b"], eps, bsh)
    y = g.output(out_name, bsh)
    g.node("Identity", dict(input=ln), bsh, out=y)
    return g.sdfg


# ---------------------------------------------------------------------------------------------
# config 4: MBConv block with folded BatchNorm
# ---------------------------------------------------------------------------------------------
def mbconv_sdfg(p, x_shape, fused=True, dtype=torch.float32):
    """``p``: ``w_exp [M,C,1,1], b_exp, w_dw [M,1,3,3], b_dw, w_se1 [R,M,1,1], b_se1, w_se2 [M,R,1,1], b_se2,
    w_proj [C,M,1,1], b_proj``."""
    n, cin, h, w = x_shape
    mid = p["w_exp"].shape[0]
    red = p["w_se1"].shape[0]
    g = GraphBuilder("mbconv", dtype)
    x = g.input("input", x_shape)
    c = {k: g.constant(k, v.to(dtype)) for k, v in p.items()}
    big, small = (n, mid, h, w), (n, mid, 1, 1)
    y = g.output("__return", x_shape)
    if fused:
        e = g.node("FusedConv", dict(X=x, W=c["w_exp"], B=c["b_exp"]), big, activation="Swish")
        dw = g.node("FusedConv", dict(X=e, W=c["w_dw"], B=c["b_dw"]), big, pads=[1, 1, 1, 1], group=mid,
                    activation="Swish")
        pool = g.extra_output(dw, "Pool", small)
        w1 = g.constant("w_se1_2d", p["w_se1"].reshape(red, mid).to(dtype))
        w2 = g.constant("w_se2_2d", p["w_se2"].reshape(mid, red).to(dtype))
        gate = g.node("SqueezeExcite", dict(X=pool, W1=w1, B1=c["b_se1"], W2=w2, B2=c["b_se2"]), small)
        g.node("FusedConv", dict(X=dw, W=c["w_proj"], B=c["b_proj"], Gate=gate, Residual=x), x_shape, out=y)
        return g.sdfg

    def swish(t, shape):
        s = g.node("Sigmoid", dict(X=t), shape)
        return g.node("Mul", dict(A=t, B=s), shape)

    e = swish(g.node("Conv", dict(X=x, W=c["w_exp"], B=c["b_exp"]), big, kernel_shape=[1, 1]), big)
    dw = swish(g.node("Conv", dict(X=e, W=c["w_dw"], B=c["b_dw"]), big, kernel_shape=[3, 3], pads=[1, 1, 1, 1],
                      group=mid), big)
    pool = g.node("GlobalAveragePool", dict(X=dw), small)
    s1 = swish(g.node("Conv", dict(X=pool, W=c["w_se1"], B=c["b_se1"]), (n, red, 1, 1), kernel_shape=[1, 1]),
               (n, red, 1, 1))
    s2 = g.node("Sigmoid", dict(X=g.node("Conv", dict(X=s1, W=c["w_se2"], B=c["b_se2"]), small, kernel_shape=[1, 1])),
                small)
    gated = g.node("Mul", dict(A=s2, B=dw), big)
    proj = g.node("Conv", dict(X=gated, W=c["w_proj"], B=c["b_proj"]), x_shape, kernel_shape=[1, 1])
    g.node("Add", dict(A=proj, B=x), x_shape, out=y)
    return g.sdfg


# ---------------------------------------------------------------------------------------------
# config 1: one strided convolution
# ---------------------------------------------------------------------------------------------
def conv_sdfg(x_shape, w_shape, strides=(1, 1), pads=(0, 0, 0, 0), bias=False, dtype=torch.float32):
    n, c, h, w = x_shape
    m, _, kh, kw = w_shape
    oh = (h + pads[0] + pads[2] - kh) // strides[0] + 1
    ow = (w + pads[1] + pads[3] - kw) // strides[1] + 1
    g = GraphBuilder("conv", dtype)
    ins = dict(X=g.input("X", x_shape), W=g.input("W", w_shape))
    if bias:
        ins["B"] = g.input("B", (m, ))
    y = g.output("Y", (n, m, oh, ow))
    g.node("Conv", ins, (n, m, oh, ow), out=y, strides=list(strides), pads=list(pads))
    return g.sdfg
