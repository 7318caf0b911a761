"""Writes the golden vectors of tests/golden/*.npz.

Run from the repository root: ``python tests/golden/generate_golden.py``.

The reference stores no golden vectors for this path and cannot be executed here (it needs DaCe to
generate its code), so each vector is produced by the CPU oracle (``oracle/ops.py``) from a seeded
input and is accepted only if an independent witness -- PyTorch's CPU operator, the comparator the
reference's own tests use (``tests/pure_expansions/test_conv_expansion.py:28-36``,
``tests/torch/test_bert_encoder.py:20-31``) -- agrees with it.  Shapes follow the reference's tests
where it has one, and small versions of the five benchmark configurations otherwise.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ops  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def witness(a, b, rtol=1e-5, atol=1e-5, what=""):
    np.testing.assert_allclose(np.asarray(a, np.float64), np.asarray(b, np.float64), rtol=rtol, atol=atol, err_msg=what)


def save(name, **arrays):
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **arrays)
    print("wrote", name, {k: v.shape for k, v in arrays.items()})


def bert_params(rng, hidden, ffn, scale=0.05):
    def w(*s):
        return (rng.standard_normal(s) * scale).astype(np.float32)
    return dict(wq=w(hidden, hidden), bq=w(hidden), wk=w(hidden, hidden), bk=w(hidden), wv=w(hidden, hidden),
                bv=w(hidden), wo=w(hidden, hidden), bo=w(hidden), ln1_g=(1 + w(hidden)), ln1_b=w(hidden),
                w1=w(ffn, hidden), b1=w(ffn), w2=w(hidden, ffn), b2=w(hidden), ln2_g=(1 + w(hidden)), ln2_b=w(hidden))


def main():
    rng = np.random.default_rng(1234)

    # MatMul: tests/pure_expansions/test_expansions.py:23-63 ([2,4] x [4,3]) plus batched forms
    a, b = rng.random((2, 4), np.float32), rng.random((4, 3), np.float32)
    y = ops.matmul(a, b)
    witness(y, a @ b)
    a3, b3 = rng.standard_normal((3, 5, 8)).astype(np.float32), rng.standard_normal((8, 6)).astype(np.float32)
    y3 = ops.matmul(a3, b3)
    witness(y3, torch.matmul(torch.from_numpy(a3), torch.from_numpy(b3)).numpy(), atol=1e-5)
    a4, b4 = rng.standard_normal((2, 3, 16, 8)).astype(np.float32), rng.standard_normal((2, 3, 8, 24)).astype(np.float32)
    y4 = ops.matmul(a4, b4)
    witness(y4, torch.matmul(torch.from_numpy(a4), torch.from_numpy(b4)).numpy(), atol=1e-5)
    save("matmul", a=a, b=b, y=y, a3=a3, b3=b3, y3=y3, a4=a4, b4=b4, y4=y4)

    # Einsum 'bij,jk->bik': test_expansions.py:387-405
    e1, e2 = rng.random((5, 3, 4), np.float32), rng.random((4, 6), np.float32)
    ye = ops.einsum("bij, jk -> bik", e1, e2)
    witness(ye, np.einsum("bij,jk->bik", e1, e2))
    save("einsum", a=e1, b=e2, y=ye)

    # Gemm: nn.Linear export (transB=1, C[N]) with alpha / beta variations
    ga, gb, gc = (rng.standard_normal((7, 12)).astype(np.float32), rng.standard_normal((5, 12)).astype(np.float32),
                  rng.standard_normal(5).astype(np.float32))
    yg = ops.gemm(ga, gb, gc, alpha=0.5, beta=2.0, trans_b=1)
    witness(yg, 0.5 * ga @ gb.T + 2.0 * gc, atol=1e-5)
    gat, gc2 = np.ascontiguousarray(ga.T), rng.standard_normal((7, 5)).astype(np.float32)
    yg2 = ops.gemm(gat, np.ascontiguousarray(gb.T), gc2, trans_a=1)
    witness(yg2, ga @ gb.T + gc2, atol=1e-5)
    save("gemm", a=ga, b=gb, c=gc, y=yg, at=gat, bt=np.ascontiguousarray(gb.T), c2=gc2, y2=yg2)

    # Reductions: test_expansions.py:187-237 on a (2,4,10) tensor scaled by 10
    rx = (rng.standard_normal((2, 4, 10)) * 10).astype(np.float32)
    red = {}
    for kind, keep, axes in [("sum", True, [0]), ("sum", False, [-1]), ("sum", True, [0, -1]), ("max", False, [0, -1]),
                             ("max", True, [0]), ("max", True, [-1]), ("mean", True, [-1]), ("mean", True, [0, -1]),
                             ("mean", False, [0]), ("min", True, [1])]:
        out = getattr(ops, "reduce_" + kind)(rx, axes, keep)
        witness(out, getattr(np, kind)(rx, axis=tuple(axes), keepdims=keep), atol=1e-5)
        red["%s_%d_%s" % (kind, int(keep), "_".join(str(a) for a in axes))] = out
    red["mean_scalar"] = ops.reduce_mean(rx, None, 0)  # test_expansions.py:240-278
    save("reduce", x=rx, **red)

    # Softmax / LogSoftmax with opset-12 axis semantics
    sx = rng.standard_normal((3, 4, 5, 16)).astype(np.float32)
    sm3 = ops.softmax(sx, axis=3)
    witness(sm3, F.softmax(torch.from_numpy(sx), -1).numpy(), atol=1e-6)
    sm1 = ops.softmax(sx, axis=1)  # joint over the last three axes
    witness(sm1, F.softmax(torch.from_numpy(sx).reshape(3, -1), -1).reshape(sx.shape).numpy(), atol=1e-6)
    ls = ops.log_softmax(sx[0, 0], axis=1)
    witness(ls, F.log_softmax(torch.from_numpy(sx[0, 0]), -1).numpy(), atol=1e-6)
    save("softmax", x=sx, softmax_axis3=sm3, softmax_axis1=sm1, logsoftmax=ls)

    # Element-wise
    ex = (rng.standard_normal((6, 33)) * 2).astype(np.float32)
    ey = (rng.standard_normal((33, )) + 3).astype(np.float32)
    ew = dict(x=ex, y=ey, add=ops.add(ex, ey), sub=ops.sub(ex, ey), mul=ops.mul(ex, ey), div=ops.div(ex, ey),
              pow2=ops.pow_(ex, np.float32(2.0)), sqrt=ops.sqrt(np.abs(ex)), erf=ops.erf(ex), exp=ops.exp(ex),
              log=ops.log(np.abs(ex) + 1), tanh=ops.tanh(ex), relu=ops.relu(ex), sigmoid=ops.sigmoid(ex),
              leaky=ops.leaky_relu(ex, 0.1), recip=ops.reciprocal(ey), softplus=ops.softplus(ex), gelu=ops.gelu_chain(ex),
              swish=ops.swish(ex), clip=ops.clip(ex, -1.0, 0.5))
    t = torch.from_numpy(ex)
    witness(ew["erf"], torch.erf(t).numpy(), atol=1e-6)
    witness(ew["gelu"], F.gelu(t).numpy(), atol=1e-6)
    witness(ew["swish"], F.silu(t).numpy(), atol=1e-6)
    witness(ew["sigmoid"], torch.sigmoid(t).numpy(), atol=1e-6)
    witness(ew["softplus"], F.softplus(t).numpy(), atol=1e-5)
    witness(ew["leaky"], F.leaky_relu(t, 0.1).numpy(), atol=1e-6)
    save("elementwise", **ew)

    # LayerNorm chain
    lx = rng.standard_normal((5, 7, 64)).astype(np.float32)
    lg, lb = (1 + 0.1 * rng.standard_normal(64)).astype(np.float32), (0.1 * rng.standard_normal(64)).astype(np.float32)
    ly = ops.layernorm_chain(lx, lg, lb, 1e-12)
    witness(ly, F.layer_norm(torch.from_numpy(lx), (64, ), torch.from_numpy(lg), torch.from_numpy(lb), 1e-12).numpy(), atol=1e-5)
    save("layernorm", x=lx, gamma=lg, beta=lb, y=ly)

    # Conv: the four cases of tests/pure_expansions/test_conv_expansion.py:9-12 (batch 8 -> 2, 32x32 -> 12x12),
    # then the strided (config 1), padded / grouped / depthwise forms the reference delegates to cuDNN
    conv = {}
    for i, (cin, ks, nf, bias) in enumerate([(1, (3, 3), 8, True), (8, (3, 3), 3, False), (8, (5, 5), 3, True), (8, (4, 4), 3, False)]):
        x = rng.random((2, cin, 12, 12), np.float32)
        w = rng.random((nf, cin) + ks, np.float32)
        b = rng.random(nf, np.float32) if bias else None
        y = ops.conv2d(x, w, b)
        witness(y, F.conv2d(torch.from_numpy(x), torch.from_numpy(w), torch.from_numpy(b) if bias else None).numpy(), atol=1e-4)
        conv.update({"x%d" % i: x, "w%d" % i: w, "y%d" % i: y})
        if bias:
            conv["b%d" % i] = b
    x = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    w = rng.random((16, 3, 3, 3), np.float32)
    y = ops.conv2d(x, w, strides=(2, 2))
    witness(y, F.conv2d(torch.from_numpy(x), torch.from_numpy(w), stride=2).numpy(), atol=1e-4)
    conv.update(xs=x, ws=w, ys=y)
    x = rng.standard_normal((2, 8, 9, 11)).astype(np.float32)
    w = rng.standard_normal((6, 4, 3, 2)).astype(np.float32)
    b = rng.standard_normal(6).astype(np.float32)
    y = ops.conv2d(x, w, b, strides=(2, 1), pads=(1, 0, 2, 1), dilations=(1, 2), group=2)
    tw = F.conv2d(F.pad(torch.from_numpy(x), (0, 1, 1, 2)), torch.from_numpy(w), torch.from_numpy(b), stride=(2, 1), dilation=(1, 2), groups=2)
    witness(y, tw.numpy(), atol=1e-4)
    conv.update(xg=x, wg=w, bg=b, yg=y)
    x = rng.standard_normal((2, 12, 10, 10)).astype(np.float32)
    w = rng.standard_normal((12, 1, 3, 3)).astype(np.float32)
    y = ops.conv2d(x, w, pads=(1, 1, 1, 1), group=12)
    witness(y, F.conv2d(torch.from_numpy(x), torch.from_numpy(w), padding=1, groups=12).numpy(), atol=1e-4)
    conv.update(xd=x, wd=w, yd=y)
    gap = ops.global_average_pool(x)
    witness(gap, torch.from_numpy(x).mean((2, 3), keepdim=True).numpy(), atol=1e-6)
    conv.update(gap=gap)
    save("conv", **conv)

    # config 2 (small): MLP
    mp = dict(w1=rng.standard_normal((24, 40)).astype(np.float32) * 0.2, b1=rng.standard_normal(24).astype(np.float32) * 0.1,
              w2=rng.standard_normal((12, 24)).astype(np.float32) * 0.2, b2=rng.standard_normal(12).astype(np.float32) * 0.1,
              w3=rng.standard_normal((10, 12)).astype(np.float32) * 0.2, b3=rng.standard_normal(10).astype(np.float32) * 0.1)
    mx = rng.standard_normal((16, 40)).astype(np.float32)
    my = ops.mlp(mx, mp)
    t = torch.from_numpy(mx)
    for i in (1, 2, 3):
        t = t @ torch.from_numpy(mp["w%d" % i]).T + torch.from_numpy(mp["b%d" % i])
        if i < 3:
            t = torch.relu(t)
    witness(my, F.log_softmax(t, -1).numpy(), atol=1e-5)
    save("mlp", x=mx, y=my, **mp)

    # config 3 (small): BERT layer, hidden 128, 2 heads of 64, FFN 256; fp32 and the fp16 storage rule
    bp = bert_params(rng, 128, 256)
    bx = rng.standard_normal((2, 40, 128)).astype(np.float32)
    by32 = ops.bert_layer(bx, bp, heads=2, store=np.float32)
    from transformers import BertConfig
    from transformers.models.bert.modeling_bert import BertLayer
    cfg = BertConfig(hidden_size=128, num_attention_heads=2, intermediate_size=256)
    cfg._attn_implementation = "eager"
    m = BertLayer(cfg).eval()
    sd = m.state_dict()
    names = {"attention.self.query": ("wq", "bq"), "attention.self.key": ("wk", "bk"), "attention.self.value": ("wv", "bv"),
             "attention.output.dense": ("wo", "bo"), "intermediate.dense": ("w1", "b1"), "output.dense": ("w2", "b2")}
    for k, (w, b) in names.items():
        sd[k + ".weight"], sd[k + ".bias"] = torch.from_numpy(bp[w]), torch.from_numpy(bp[b])
    sd["attention.output.LayerNorm.weight"], sd["attention.output.LayerNorm.bias"] = torch.from_numpy(bp["ln1_g"]), torch.from_numpy(bp["ln1_b"])
    sd["output.LayerNorm.weight"], sd["output.LayerNorm.bias"] = torch.from_numpy(bp["ln2_g"]), torch.from_numpy(bp["ln2_b"])
    m.load_state_dict(sd)
    with torch.no_grad():
        hf = m(torch.from_numpy(bx))
    hf = hf[0] if isinstance(hf, tuple) else hf
    witness(by32, hf.numpy(), atol=2e-5, what="bert layer vs HuggingFace BertLayer")
    by16 = ops.bert_layer(bx, bp, heads=2, store=np.float16)
    save("bert_layer", x=bx, y_fp32=by32, y_fp16=by16.astype(np.float32), **bp)

    # config 4 (small): MBConv block
    cp = dict(w_exp=rng.standard_normal((24, 8, 1, 1)).astype(np.float32) * 0.2, b_exp=rng.standard_normal(24).astype(np.float32) * 0.1,
              w_dw=rng.standard_normal((24, 1, 3, 3)).astype(np.float32) * 0.2, b_dw=rng.standard_normal(24).astype(np.float32) * 0.1,
              w_se1=rng.standard_normal((4, 24, 1, 1)).astype(np.float32) * 0.2, b_se1=rng.standard_normal(4).astype(np.float32) * 0.1,
              w_se2=rng.standard_normal((24, 4, 1, 1)).astype(np.float32) * 0.2, b_se2=rng.standard_normal(24).astype(np.float32) * 0.1,
              w_proj=rng.standard_normal((8, 24, 1, 1)).astype(np.float32) * 0.2, b_proj=rng.standard_normal(8).astype(np.float32) * 0.1)
    cx = rng.standard_normal((3, 8, 12, 12)).astype(np.float32)
    cy = ops.mbconv_block(cx, cp)
    tp = {k: torch.from_numpy(v) for k, v in cp.items()}
    t = torch.from_numpy(cx)
    h = F.silu(F.conv2d(t, tp["w_exp"], tp["b_exp"]))
    h = F.silu(F.conv2d(h, tp["w_dw"], tp["b_dw"], padding=1, groups=24))
    s = h.mean((2, 3), keepdim=True)
    s = F.silu(F.conv2d(s, tp["w_se1"], tp["b_se1"]))
    s = torch.sigmoid(F.conv2d(s, tp["w_se2"], tp["b_se2"]))
    ty = F.conv2d(s * h, tp["w_proj"], tp["b_proj"]) + t
    witness(cy, ty.numpy(), atol=1e-5)
    save("mbconv", x=cx, y=cy, **cp)


if __name__ == "__main__":
    main()
