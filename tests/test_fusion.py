"""The fusion pass: exported (node-for-node) graphs collapse into the fused operators, and only where that is safe."""
import numpy as np
import pytest
import torch

import daceml_b200.onnx as donnx
from daceml_b200 import graphs, sdfg as sd
from daceml_b200.transformation import fuse_subgraphs, patterns
from daceml_b200.util.utils import auto_optimize


def rn(gen, *s):
    return torch.randn(*s, generator=gen) * 0.02


def bert_params(gen, H, F_):
    return dict(wq=rn(gen, H, H), bq=rn(gen, H), wk=rn(gen, H, H), bk=rn(gen, H), wv=rn(gen, H, H), bv=rn(gen, H), wo=rn(gen, H, H),
                bo=rn(gen, H), ln1_g=torch.ones(H), ln1_b=torch.zeros(H), w1=rn(gen, F_, H), b1=rn(gen, F_), w2=rn(gen, H, F_),
                b2=rn(gen, H), ln2_g=torch.ones(H), ln2_b=torch.zeros(H))


def kinds(s):
    out = []
    for n in s.states()[0].topological_compute_nodes():
        tag = type(n).schema.name
        if getattr(n, "activation", ""):
            tag += ":" + n.activation
        if getattr(n, "ln_epsilon", None) is not None:
            tag += ":ln"
        out.append(tag)
    return out


@pytest.mark.parametrize("with_mask", [False, True])
def test_exported_bert_layer_collapses_to_five_nodes(with_mask):
    gen = torch.Generator().manual_seed(0)
    p = bert_params(gen, 256, 512)
    if with_mask:
        p["mask"] = torch.zeros(2, 128)
    s = graphs.bert_layer_sdfg(p, 2, 128, 4, fused=False)
    assert len(kinds(s)) == (58 if with_mask else 56)
    assert fuse_subgraphs(s) > 0
    assert kinds(s) == ["FusedMatMul", "Attention", "FusedMatMul:ln", "FusedMatMul:Gelu", "FusedMatMul:ln"]
    assert kinds(s) == kinds(graphs.bert_layer_sdfg(p, 2, 128, 4, fused=True))
    att = next(n for n in s.states()[0].nodes() if isinstance(n, donnx.ONNXAttention))
    assert att.num_heads == 4 and abs(att.scale - 0.125) < 1e-6
    # the three projections were packed: one [768, 256] weight, Attention reads the packed tensor
    assert not any(True for _ in s.states()[0].in_edges_by_connector(att, "K"))
    assert any(tuple(t.shape) == (768, 256) for t in s.constants.values())
    # dead intermediates and their scalar constants are gone
    assert fuse_subgraphs(s) == 0
    assert len([a for a, d in s.arrays.items() if d.transient]) == 4


def test_exported_mlp_and_mbconv_collapse():
    gen = torch.Generator().manual_seed(1)
    mp = dict(w1=rn(gen, 120, 784), b1=rn(gen, 120), w2=rn(gen, 32, 120), b2=rn(gen, 32), w3=rn(gen, 10, 32), b3=rn(gen, 10))
    s = graphs.mlp_sdfg(mp, 64, fused=False)
    auto_optimize(s, cuda=True)
    assert [t.kernels for t in s.states()[0].topological_compute_nodes()] == [("gemm", ), ("gemm", ), ("gemm", ), ("softmax", )]
    cp = dict(w_exp=rn(gen, 144, 24, 1, 1), b_exp=rn(gen, 144), w_dw=rn(gen, 144, 1, 3, 3), b_dw=rn(gen, 144), w_se1=rn(gen, 6, 144, 1, 1),
              b_se1=rn(gen, 6), w_se2=rn(gen, 144, 6, 1, 1), b_se2=rn(gen, 144), w_proj=rn(gen, 24, 144, 1, 1), b_proj=rn(gen, 24))
    s = graphs.mbconv_sdfg(cp, (4, 24, 56, 56), fused=False)
    assert len(kinds(s)) == 15
    fuse_subgraphs(s)
    assert kinds(s) == ["FusedConv:Swish", "FusedConv:Swish", "SqueezeExcite", "FusedConv"]
    proj = [n for n in s.states()[0].topological_compute_nodes()][-1]
    conns = {e.dst_conn for e in s.states()[0].in_edges(proj)}
    assert {"X", "W", "B", "Gate", "Residual"} <= conns


def test_intermediates_with_other_readers_are_not_fused():
    """A GELU chain whose Erf output is also a graph output must stay as it is."""
    g = graphs.GraphBuilder("keep", torch.float32)
    x = g.input("x", (4, 8))
    d = g.node("Div", dict(A=x, B=g.scalar(1.41421354)), (4, 8))
    e_out = g.output("erf_out", (4, 8))
    g.node("Erf", dict(input=d), (4, 8), out=e_out)
    a = g.node("Add", dict(A=e_out, B=g.scalar(1.0)), (4, 8))
    m = g.node("Mul", dict(A=x, B=a), (4, 8))
    y = g.output("y", (4, 8))
    g.node("Mul", dict(A=m, B=g.scalar(0.5)), (4, 8), out=y)
    assert patterns.fuse_gelu(g.sdfg) == 0
    assert len(kinds(g.sdfg)) == 5


def test_layernorm_pattern_needs_last_axis_and_constants():
    g = graphs.GraphBuilder("ln", torch.float32)
    x = g.input("x", (4, 6, 8))
    gamma, beta = g.constant("gamma", torch.ones(8)), g.constant("beta", torch.zeros(8))
    y = graphs._layernorm_chain(g, x, gamma, beta, 1e-5, (4, 6, 8))
    out = g.output("__return", (4, 6, 8))
    g.node("Identity", dict(input=y), (4, 6, 8), out=out)
    s = g.sdfg
    fuse_subgraphs(s)
    assert kinds(s) == ["LayerNormalization"]
    ln = s.states()[0].topological_compute_nodes()[0]
    assert abs(ln.epsilon - 1e-5) < 1e-12
    # reduction over another axis: not a LayerNorm over rows, left alone
    g2 = graphs.GraphBuilder("ln2", torch.float32)
    x2 = g2.input("x", (4, 6, 8))
    mean = g2.node("ReduceMean", dict(data=x2), (4, 1, 8), axes=[1], keepdims=1)
    out2 = g2.output("__return", (4, 6, 8))
    g2.node("Sub", dict(A=x2, B=mean), (4, 6, 8), out=out2)
    assert fuse_subgraphs(g2.sdfg) == 0


def _attention_block(g, x, mask4, batch, seq, heads, d, out_name):
    """The exported attention sub-graph on one [B, S, H] input (Q = K = V = x), with an additive mask operand."""
    hidden = heads * d

    def split(perm):
        r = g.node("Reshape", dict(data=x), (batch, seq, heads, d))
        return g.node("Transpose", dict(data=r), tuple((batch, seq, heads, d)[i] for i in perm), perm=list(perm))

    q, k, v = split((0, 2, 1, 3)), split((0, 2, 3, 1)), split((0, 2, 1, 3))
    s = g.node("MatMul", dict(A=q, B=k), (batch, heads, seq, seq))
    s = g.node("Mul", dict(A=s, B=g.scalar(0.125)), (batch, heads, seq, seq))
    s = g.node("Add", dict(A=s, B=mask4), (batch, heads, seq, seq))
    p = g.node("Softmax", dict(input=s), (batch, heads, seq, seq), axis=3)
    c = g.node("MatMul", dict(A=p, B=v), (batch, heads, seq, d))
    c = g.node("Transpose", dict(data=c), (batch, seq, heads, d), perm=[0, 2, 1, 3])
    g.node("Reshape", dict(data=c), (batch, seq, hidden), out=g.output(out_name, (batch, seq, hidden)))


@pytest.mark.parametrize("mask_shape, reshaped", [((1, 128), (1, 1, 1, 128)), ((128, 128), (1, 1, 128, 128)),
                                                  ((2, 128), (2, 1, 1, 128))])
def test_attention_fusion_takes_only_per_batch_key_masks(mask_shape, reshaped):
    """The fused kernel reads its mask as [batch, keys]: a row broadcast over the batch or a [S, S] bias is not one."""
    g = graphs.GraphBuilder("att", torch.float16)
    x = g.input("x", (2, 128, 256))
    m = g.constant("mask", torch.zeros(mask_shape, dtype=torch.float16))
    m4 = g.node("Reshape", dict(data=m), reshaped)
    _attention_block(g, x, m4, 2, 128, 4, 64, "__return")
    fused = patterns.fuse_attention(g.sdfg)
    if mask_shape == (2, 128):
        assert fused == 1 and kinds(g.sdfg) == ["Attention"]
    else:
        assert fused == 0 and "Softmax" in kinds(g.sdfg) and "Add" in kinds(g.sdfg)


def test_attention_fusion_keeps_a_mask_reshape_other_layers_read():
    """One constant mask, reshaped once, added to the scores of two attention blocks: both fuse, and neither is left
    reading an array whose producer was removed."""
    g = graphs.GraphBuilder("att2", torch.float16)
    x1, x2 = g.input("x1", (2, 128, 256)), g.input("x2", (2, 128, 256))
    m = g.constant("mask", torch.zeros(2, 128, dtype=torch.float16))
    m4 = g.node("Reshape", dict(data=m), (2, 1, 1, 128))
    _attention_block(g, x1, m4, 2, 128, 4, 64, "__return_0")
    _attention_block(g, x2, m4, 2, 128, 4, 64, "__return_1")
    s = g.sdfg
    assert fuse_subgraphs(s) > 0
    assert sorted(kinds(s)) == ["Attention", "Attention"]
    st = s.states()[0]
    for att in st.topological_compute_nodes():
        mask = next(e.data.data for e in st.in_edges_by_connector(att, "Mask"))
        assert mask in s.constants and tuple(s.constants[mask].shape) == (2, 128)
