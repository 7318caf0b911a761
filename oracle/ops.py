"""CPU oracle: a numpy restatement of DaCeML's "pure" ONNX operator expansions.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path (``daceml_b200/``) imports this module;
it is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of
``bench.py``.

Each function follows the reference expansion it cites (paths are relative to the reference
project).  The reference's own arithmetic is produced by DaCe's code generator
(``git+https://github.com/spcl/dace.git@backport-0.13-fixes``, ``setup.py:40``), which is not
vendored and cannot be installed here, so the reference itself cannot be executed.  The oracle is
pinned the way the reference's tests pin the expansions: against numpy / PyTorch on the shapes of
``tests/pure_expansions/test_expansions.py`` and ``tests/pure_expansions/test_conv_expansion.py``
(the reference stores no golden vectors for this path; it compares against numpy / torch on fresh
random inputs).  fp16, strided convolution and depthwise convolution have no pure expansion and no
test in the reference: for those the oracle is the ONNX definition and parity is unpinned.

Precision rule (``daceml/transformation/mixed_precision.py:5-35``): tensors between nodes keep
their storage type; anything written through a reduction is accumulated in fp32.  The oracle
therefore computes in fp32 (fp64 where noted) from inputs already rounded to the storage type.
"""
import itertools
import math

import numpy as np

try:  # scipy is present in the image; fall back to math.erf for a bare numpy install
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf, otypes=[np.float64])


# ---------------------------------------------------------------------------------------------
# MatMul / Einsum / Gemm
# ---------------------------------------------------------------------------------------------
def matmul_equation(a_shape, b_shape, trans_a=False, trans_b=False):
    """The einsum string PureMatMul / PureGemm build (pure_implementations.py:129-197, 398-458).

    The last two dimensions are ``ik,kj->ij``; walking the leading dimensions of both operands
    from the right, a dimension present in both gets one shared letter, a dimension present in one
    operand only gets a letter on that operand and on the result.  Letters are popped from
    ``z..a`` without ``i, j, k``.  transA / transB reverse the operand's subscript string."""
    letters = [chr(ord('z') - i) for i in range(26)]
    letters = [l for l in letters if l not in ('i', 'j', 'k')]
    if len(a_shape) == 1:
        if len(b_shape) != 2:
            raise ValueError("invalid dimensions")
        arg1, arg2, result = 'k', 'kj', 'j'
    elif len(b_shape) == 1:
        if len(a_shape) != 2:
            raise ValueError("invalid dimensions")
        arg1, arg2, result = 'ik', 'k', 'i'
    else:
        arg1, arg2, result = 'ik', 'kj', 'ij'
        for dim0, dim1 in itertools.zip_longest(reversed(a_shape[:-2]), reversed(b_shape[:-2])):
            letter = letters.pop()
            if dim0 is None:
                arg2, result = letter + arg2, letter + result
            elif dim1 is None:
                arg1, result = letter + arg1, letter + result
            else:
                arg1, arg2, result = letter + arg1, letter + arg2, letter + result
    if trans_a:
        arg1 = ''.join(reversed(arg1))
    if trans_b:
        arg2 = ''.join(reversed(arg2))
    return '{},{}->{}'.format(arg1, arg2, result)


def einsum(equation, *inputs, acc_dtype=np.float32):
    """PureEinsum (pure_implementations.py:219-252): spaces removed, '...' rejected."""
    equation = equation.replace(" ", "")
    if "..." in equation:
        raise ValueError("ellipsis is not supported by the pure Einsum expansion")
    out_dtype = inputs[0].dtype
    res = np.einsum(equation, *[np.asarray(x, dtype=acc_dtype) for x in inputs], optimize=True)
    return res.astype(out_dtype)


def matmul(a, b, acc_dtype=np.float32):
    """PureMatMul (pure_implementations.py:111-216); 1-D operands are rejected (:116-121)."""
    if a.ndim == 1 or b.ndim == 1:
        raise ValueError("the pure MatMul expansion rejects 1-D operands")
    return einsum(matmul_equation(a.shape, b.shape), a, b, acc_dtype=acc_dtype)


def gemm(a, b, c=None, alpha=1.0, beta=1.0, trans_a=0, trans_b=0, acc_dtype=np.float32):
    """PureGemm (pure_implementations.py:380-553): Y = alpha * op(A) op(B) + beta * C.

    C is indexed by the last ``len(C.shape)`` result indices and every C dimension must equal
    the matching Y dimension (:533-539); a C of shape [1, N] or a scalar raises ValueError."""
    eq = matmul_equation(a.shape, b.shape, bool(trans_a), bool(trans_b))
    y = np.einsum(eq, np.asarray(a, dtype=acc_dtype), np.asarray(b, dtype=acc_dtype), optimize=True)
    if alpha != 1:
        y = y * acc_dtype(alpha)
    if beta != 0 and c is not None:
        for c_shp, y_shp in zip(reversed(c.shape), reversed(y.shape)):
            if c_shp != y_shp:
                raise ValueError('Could not broadcast dimensions from C to Y in ONNXGemm')
        cc = np.asarray(c, dtype=acc_dtype)
        y = y + (cc if beta == 1 else cc * acc_dtype(beta))
    return y.astype(a.dtype)


# ---------------------------------------------------------------------------------------------
# Softmax family (opset <= 12 semantics)
# ---------------------------------------------------------------------------------------------
def _softmax_axes(x, axis):
    return tuple(list(range(x.ndim))[axis:])


def softmax(x, axis=1):
    """Softmax (pure_implementations.py:304-319): reduce jointly over all axes from ``axis`` on."""
    axes = _softmax_axes(x, axis)
    xf = np.asarray(x, dtype=np.float32)
    maximum = np.maximum.reduce(xf, axis=axes, keepdims=True)
    exponent = np.exp(xf - maximum)
    total = np.add.reduce(exponent, axis=axes, keepdims=True)
    return (exponent / total).astype(x.dtype)


def log_softmax(x, axis=1):
    """LogSoftmax (pure_implementations.py:649-656): x - max - log(sum(exp(x - max)))."""
    axes = _softmax_axes(x, axis)
    xf = np.asarray(x, dtype=np.float32)
    maximum = np.maximum.reduce(xf, axis=axes, keepdims=True)
    max_sub = xf - maximum
    exponent = np.exp(max_sub)
    total = np.add.reduce(exponent, axis=axes, keepdims=True)
    return (max_sub - np.log(total)).astype(x.dtype)


# ---------------------------------------------------------------------------------------------
# Element-wise (numpy broadcasting; pure_implementations.py:24-108, 283-291, 556-568, 736-743)
# ---------------------------------------------------------------------------------------------
def _f(x):
    return np.asarray(x, dtype=np.float32)


def _binary(fn, a, b):
    out_dtype = np.result_type(a.dtype, b.dtype) if hasattr(b, "dtype") else a.dtype
    return fn(_f(a), _f(b)).astype(out_dtype)


def add(a, b): return _binary(np.add, a, b)            # :76-78
def sub(a, b): return _binary(np.subtract, a, b)       # :81-83
def mul(a, b): return _binary(np.multiply, a, b)       # :86-88
def div(a, b): return _binary(np.divide, a, b)         # :91-93
def pow_(a, b): return _binary(np.power, a, b)         # :39-41


def sqrt(x): return np.sqrt(_f(x)).astype(x.dtype)      # :34-36
def exp(x): return np.exp(_f(x)).astype(x.dtype)        # :29-31
def log(x): return np.log(_f(x)).astype(x.dtype)        # :24-26
def tanh(x): return np.tanh(_f(x)).astype(x.dtype)      # :289-291
def erf(x): return _erf(np.asarray(x, dtype=np.float64)).astype(x.dtype)  # :106-108
def relu(x): return np.maximum(_f(x), 0).astype(x.dtype)                   # :556-560
def reciprocal(x): return (np.float32(1) / _f(x)).astype(x.dtype)          # :283-286
def identity(x): return np.array(x, copy=True)                             # :255-257


def leaky_relu(x, alpha=0.01):  # :563-568
    xf = _f(x)
    return (np.maximum(xf, 0) + np.float32(alpha) * np.minimum(xf, 0)).astype(x.dtype)


def sigmoid(x):  # :741-743
    return (np.float32(1) / (np.float32(1) + np.exp(-_f(x)))).astype(x.dtype)


def softplus(x):  # :736-738
    return np.log(np.float32(1) + np.exp(_f(x))).astype(x.dtype)


def clip(x, lo, hi):  # :44-73
    return np.minimum(np.maximum(_f(x), np.float32(lo)), np.float32(hi)).astype(x.dtype)


def cast(x, dtype):  # :329-377
    return np.asarray(x).astype(dtype)


# ---------------------------------------------------------------------------------------------
# Reductions (pure_implementations.py:101-103, 294-306); the output descriptor carries keepdims
# ---------------------------------------------------------------------------------------------
def _reduce(fn, x, axes, keepdims):
    ax = None if axes is None else tuple(int(a) for a in axes)
    return fn(_f(x), axis=ax, keepdims=bool(keepdims)).astype(x.dtype)


def reduce_mean(x, axes=None, keepdims=1): return _reduce(np.mean, x, axes, keepdims)
def reduce_sum(x, axes=None, keepdims=1): return _reduce(np.sum, x, axes, keepdims)
def reduce_max(x, axes=None, keepdims=1): return _reduce(np.max, x, axes, keepdims)
def reduce_min(x, axes=None, keepdims=1): return _reduce(np.min, x, axes, keepdims)


# ---------------------------------------------------------------------------------------------
# Data movement (pure_implementations.py:322-326, 571-581, 746-778, 1016-1026)
# ---------------------------------------------------------------------------------------------
def transpose(x, perm=None):
    return np.ascontiguousarray(np.transpose(x, axes=perm if perm is not None else list(reversed(range(x.ndim)))))


def reshape(x, shape):
    return np.reshape(x, shape)


def flatten(x, axis=1):
    return x.reshape([int(np.prod(x.shape[:axis], dtype=np.int64)), int(np.prod(x.shape[axis:], dtype=np.int64))])


def unsqueeze(x, axes):
    out = x
    for a in sorted(axes):
        out = np.expand_dims(out, a)
    return out


def shape(x):  # :907-946
    return np.array(x.shape, dtype=np.int64)


def gather(data, indices, axis=0):
    """PureGather (:949-1014): "read the docs for np.take"; the output is indexed by
    ``data.shape[:axis] + indices.shape + data.shape[axis+1:]`` and element ``[.., j.., ..]`` reads
    ``data[.., indices[j..], ..]``.  Restated as loops over the index tensor rather than by calling np.take."""
    data, indices = np.asarray(data), np.asarray(indices, dtype=np.int64)
    axis %= data.ndim
    out = np.empty(data.shape[:axis] + indices.shape + data.shape[axis + 1:], dtype=data.dtype)
    lead = (slice(None), ) * axis
    for j in np.ndindex(*indices.shape):
        i = int(indices[j])
        if i < 0:
            i += data.shape[axis]
        out[lead + j] = data[lead + (i, )]
    return out


def slice_(data, starts, ends, axes=None, steps=None):
    """ONNX Slice-10 with constant index inputs.  The reference expansion (:659-735, 830-904) takes the
    ``axis 0, step 1`` case, ``output = data[start:end:1, :]``, and reads an ``INT64_MAX`` end (an exporter
    artefact) as "to the end"; this is the same rule for every axis and any positive step."""
    axes = list(range(len(starts))) if axes is None else [int(a) % data.ndim for a in axes]
    steps = [1] * len(starts) if steps is None else list(steps)
    index = [slice(None)] * data.ndim
    for s, e, a, st in zip(starts, ends, axes, steps):
        n = data.shape[a]
        s = max(0, min(n, int(s) + n if s < 0 else int(s)))
        e = max(0, min(n, int(e) + n if e < 0 else int(e)))
        index[a] = slice(s, max(s, e), int(st))
    return np.ascontiguousarray(data[tuple(index)])


def split(x, axis=0, sizes=None, parts=None):
    """SplitPure (:781-827): consecutive sub-ranges of ``axis`` with the extents of the ``split`` attribute."""
    axis %= x.ndim
    if sizes is None:
        sizes = [x.shape[axis] // parts] * parts
    outs, off = [], 0
    for n in sizes:
        index = [slice(None)] * x.ndim
        index[axis] = slice(off, off + n)
        outs.append(np.ascontiguousarray(x[tuple(index)]))
        off += n
    return outs


def concat(xs, axis):
    """ONNX Concat (the inverse of Split; the reference has no pure expansion for it)."""
    axis %= xs[0].ndim
    out = np.empty(xs[0].shape[:axis] + (sum(x.shape[axis] for x in xs), ) + xs[0].shape[axis + 1:], dtype=xs[0].dtype)
    off = 0
    for x in xs:
        index = [slice(None)] * out.ndim
        index[axis] = slice(off, off + x.shape[axis])
        out[tuple(index)] = x
        off += x.shape[axis]
    return out


def expand(x, shape):
    """ONNX Expand: numpy broadcasting of ``x`` against ``shape``.  PureExpand (:260-281) only takes the case
    where nothing changes (``output[:] = input``)."""
    return np.ascontiguousarray(np.broadcast_to(x, np.broadcast_shapes(x.shape, tuple(shape))))


def where(condition, x, y):  # :96-98, ``output[:] = np.where(condition, X, Y)``
    return np.where(condition, x, y).astype(np.result_type(x, y))


# ---------------------------------------------------------------------------------------------
# Convolution and pooling (img_op_implementations.py)
# ---------------------------------------------------------------------------------------------
def maxpool2d(x, kernel, strides=(1, 1), pads=(0, 0, 0, 0)):
    """PureMaxPool2D (img_op_implementations.py:28-161): ``Y[b, c, ox, oy]`` starts at the lowest value of the type
    and takes ``max`` over ``X[b, c, ox * stride + hx, oy * stride + hy]`` for the window.  The reference accepts no
    padding; with ONNX padding (added here) the padded positions simply never enter the maximum."""
    n, c, h, w = x.shape
    kh, kw = kernel
    oh = (h + pads[0] + pads[2] - kh) // strides[0] + 1
    ow = (w + pads[1] + pads[3] - kw) // strides[1] + 1
    y = np.full((n, c, oh, ow), np.finfo(x.dtype).min, dtype=x.dtype)
    for oy in range(oh):
        for ox in range(ow):
            for ky in range(kh):
                iy = oy * strides[0] - pads[0] + ky
                if iy < 0 or iy >= h:
                    continue
                for kx in range(kw):
                    ix = ox * strides[1] - pads[1] + kx
                    if ix < 0 or ix >= w:
                        continue
                    y[:, :, oy, ox] = np.maximum(y[:, :, oy, ox], x[:, :, iy, ix])
    return y


def conv_pure_supported(x_shape, w_shape, strides, pads, dilations, group):
    """The preconditions of PureConv2D.forward_can_be_applied (img_op_implementations.py:168-214)."""
    return (len(x_shape) == 4 and len(w_shape) == 4 and group == 1 and w_shape[1] == x_shape[1]
            and all(d == 1 for d in dilations) and all(p == 0 for p in pads) and all(s == 1 for s in strides))


def conv2d(x, w, b=None, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1):
    """ONNX Conv, NCHW cross-correlation.

    For stride 1 / no padding / group 1 this is PureConv2D (img_op_implementations.py:217-288):
    Y is initialised with the bias (or zero) and W[m,c,i,j] * X[b,c,y+i,x+j] is accumulated in
    (c, i, j) order.  Strides, pads, dilations and groups generalise the index expression per the
    ONNX definition, which the reference obtains from cuDNN in CUDNN_CROSS_CORRELATION mode
    (cudnn_implementations.py:241-275).  ``pads`` is (top, left, bottom, right)."""
    n, c, h, wd = x.shape
    m, cg, kh, kw = w.shape
    sh, sw = strides
    pt, pl, pb, pr = pads
    dh, dw = dilations
    if c % group or m % group or cg != c // group:
        raise ValueError("conv: channels do not match the group count")
    oh = (h + pt + pb - dh * (kh - 1) - 1) // sh + 1
    ow = (wd + pl + pr - dw * (kw - 1) - 1) // sw + 1
    xp = np.zeros((n, c, h + pt + pb, wd + pl + pr), dtype=np.float32)
    xp[:, :, pt:pt + h, pl:pl + wd] = x
    wf = np.asarray(w, dtype=np.float32)
    y = np.zeros((n, m, oh, ow), dtype=np.float32)
    if b is not None:
        y += np.asarray(b, dtype=np.float32)[None, :, None, None]
    mg = m // group
    for g in range(group):
        for ci in range(cg):
            for i in range(kh):
                for j in range(kw):
                    patch = xp[:, g * cg + ci, i * dh:i * dh + (oh - 1) * sh + 1:sh, j * dw:j * dw + (ow - 1) * sw + 1:sw]
                    y[:, g * mg:(g + 1) * mg] += wf[None, g * mg:(g + 1) * mg, ci, i, j, None, None] * patch[:, None]
    return y.astype(x.dtype)


def batchnorm_inference(x, scale, b, mean, var, eps=1e-5):
    """ONNX BatchNormalization, inference form: ``(x - mean) / sqrt(var + eps) * scale + b`` per channel (axis 1).
    The reference only has the training form (img_op_implementations.py:333-393, which also updates the running
    statistics); this is the ONNX definition, checked against ``torch.nn.functional.batch_norm`` in the tests."""
    bshape = (1, -1) + (1, ) * (x.ndim - 2)
    xf = np.asarray(x, dtype=np.float32)
    y = (xf - mean.reshape(bshape)) / np.sqrt(var.reshape(bshape) + np.float32(eps)) * scale.reshape(bshape) + b.reshape(bshape)
    return y.astype(x.dtype)


def global_average_pool(x):
    """GlobalAveragePool (img_op_implementations.py:415-417): mean over H, W into [N, C, 1, 1]."""
    return np.mean(_f(x), axis=(2, 3), keepdims=True).astype(x.dtype)


# ---------------------------------------------------------------------------------------------
# Node chains as the ONNX exporter emits them (opset 12 has no LayerNormalization / Gelu)
# ---------------------------------------------------------------------------------------------
def layernorm_chain(x, gamma, beta, eps=1e-12):
    """ReduceMean -> Sub -> Pow(2) -> ReduceMean -> Add(eps) -> Sqrt -> Div -> Mul -> Add."""
    xf = _f(x)
    mean = np.mean(xf, axis=-1, keepdims=True)
    d = xf - mean
    var = np.mean(np.power(d, np.float32(2.0)), axis=-1, keepdims=True)
    y = d / np.sqrt(var + np.float32(eps))
    return (y * _f(gamma) + _f(beta)).astype(x.dtype)


def gelu_chain(x):
    """Div(1.41421354) -> Erf -> Add(1) -> Mul(x) -> Mul(0.5)."""
    xf = _f(x)
    e = _erf((xf / np.float32(1.41421354)).astype(np.float64)).astype(np.float32)
    return (xf * (e + np.float32(1.0)) * np.float32(0.5)).astype(x.dtype)


def swish(x):
    """Sigmoid followed by Mul."""
    xf = _f(x)
    return (xf * (np.float32(1) / (np.float32(1) + np.exp(-xf)))).astype(x.dtype)


# ---------------------------------------------------------------------------------------------
# Whole graphs of the benchmark configurations
# ---------------------------------------------------------------------------------------------
def mlp(x, params):
    """Gemm(transB=1) -> Relu -> Gemm -> Relu -> Gemm -> LogSoftmax(axis=1)."""
    h = relu(gemm(x, params["w1"], params["b1"], trans_b=1))
    h = relu(gemm(h, params["w2"], params["b2"], trans_b=1))
    h = gemm(h, params["w3"], params["b3"], trans_b=1)
    return log_softmax(h, axis=1)


def bert_layer(x, p, heads, eps=1e-12, store=np.float16, intermediates=None):
    """The opset-12 export of a post-LN BERT encoder layer, node by node.

    Weights are nn.Linear ``[out, in]`` matrices: each appears as Transpose(W) -> MatMul -> Add(bias).
    ``store`` is the storage type between nodes (the fp16 rule); accumulation is fp32."""
    def st(t):
        return np.asarray(t, dtype=np.float32).astype(store)

    def rec(name, t):
        if intermediates is not None:
            intermediates[name] = t
        return t

    b, s, hid = x.shape
    d = hid // heads
    x = st(x)

    def linear(inp, w, bias):
        return st(add(st(matmul(inp, transpose(st(w), [1, 0]))), st(bias)))

    def split(t):
        return transpose(reshape(t, (b, s, heads, d)), [0, 2, 1, 3])

    q = split(linear(x, p["wq"], p["bq"]))
    k = split(linear(x, p["wk"], p["bk"]))
    v = split(linear(x, p["wv"], p["bv"]))
    scores = st(matmul(q, transpose(k, [0, 1, 3, 2])))
    scores = st(mul(scores, np.asarray(1.0 / math.sqrt(d), dtype=store)))
    if p.get("mask") is not None:
        scores = st(add(scores, st(p["mask"])[:, None, None, :]))
    probs = rec("probs", st(softmax(scores, axis=3)))
    ctx = st(matmul(probs, v))
    ctx = rec("context", reshape(transpose(ctx, [0, 2, 1, 3]), (b, s, hid)))
    attn = st(add(linear(ctx, p["wo"], p["bo"]), x))
    h1 = rec("attn_ln", st(layernorm_chain(attn, st(p["ln1_g"]), st(p["ln1_b"]), eps)))
    inter = rec("gelu", st(gelu_chain(linear(h1, p["w1"], p["b1"]))))
    out = st(add(linear(inter, p["w2"], p["b2"]), h1))
    return st(layernorm_chain(out, st(p["ln2_g"]), st(p["ln2_b"]), eps))


def mbconv_block(x, p):
    """EfficientNet-B0 style MBConv block with BatchNorm folded into the convolutions:
    1x1 expand -> Swish -> depthwise 3x3 (pad 1) -> Swish -> squeeze-excite -> 1x1 project -> + x."""
    c_mid = p["w_exp"].shape[0]
    h = swish(conv2d(x, p["w_exp"], p["b_exp"]))
    h = swish(conv2d(h, p["w_dw"], p["b_dw"], pads=(1, 1, 1, 1), group=c_mid))
    s = global_average_pool(h)
    s = swish(conv2d(s, p["w_se1"], p["b_se1"]))
    s = sigmoid(conv2d(s, p["w_se2"], p["b_se2"]))
    h = mul(s, h)
    return add(conv2d(h, p["w_proj"], p["b_proj"]), x)
