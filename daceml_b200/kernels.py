"""Tensor-level wrappers over the C ABI: torch tensors in, kernel launches on the current stream out.

PyTorch is used for device memory and streams only; every function here ends in exactly one call
into ``libdaceml_b200.so`` and raises when that call fails.  Outputs are pre-allocated by the
caller (as the reference's dispatchers do, ``daceml/torch/dispatchers/ctypes_module.py:58-67``).
"""
import ctypes

import torch

from . import lib as L


def _ctx(t):
    if not t.is_cuda:
        raise L.B200Error(L.ERR_INVALID, "daceml_b200 kernels need CUDA tensors; there is no CPU path")
    return L.get_context(t.device)


def _stream(t):
    return L.current_stream(t.device)


def _i64(vals):
    return (ctypes.c_int64 * len(vals))(*[int(v) for v in vals])


def _i32(vals):
    return (ctypes.c_int32 * len(vals))(*[int(v) for v in vals])


def _contig(t, name):
    if t is not None and not t.is_contiguous():
        raise L.B200Error(L.ERR_INVALID, f"{name} must be contiguous")


def gemm_raw(ctx, params, stream):
    L.check(ctx.lib.b200ml_gemm(ctx.handle, ctypes.byref(params), stream))


def gemm(a, b, out, *, b_layout=0, a_layout=0, bias=None, residual=None, act=0, alpha=1.0, bias_scale=1.0,
         residual_scale=1.0, ln=None, b_constant=False):
    """out[M,N] = act(alpha * A.B + bias_scale * bias) + residual_scale * residual for 2-D operands;
    with ``ln=(gamma, beta, eps)`` the rows of that result are layer-normalised before they are stored.

    ``a`` is [M,K] (or [K,M] with ``a_layout=1``), ``b`` is [K,N] (``b_layout=0``) or [N,K]
    (``b_layout=1``); rows may be strided (last dimension contiguous).  ``b_constant``: nothing enqueued earlier on
    the stream writes ``b`` (a weight), so the kernel may fetch it before the preceding kernel has finished."""
    ctx = _ctx(a)
    p = L.GemmParams()
    p.dtype = L.dtype_code(a.dtype)
    p.flags = L.GEMM_B_CONSTANT if b_constant else 0
    p.a_layout, p.b_layout = a_layout, b_layout
    m, k = (a.shape[0], a.shape[1]) if a_layout == 0 else (a.shape[1], a.shape[0])
    n = b.shape[1] if b_layout == 0 else b.shape[0]
    kb = b.shape[0] if b_layout == 0 else b.shape[1]
    if kb != k or tuple(out.shape) != (m, n):
        raise L.B200Error(L.ERR_INVALID, f"gemm: shape mismatch A{tuple(a.shape)} B{tuple(b.shape)} C{tuple(out.shape)}")
    for t, nm in ((a, "A"), (b, "B"), (out, "C"), (residual, "residual")):
        if t is not None and t.stride(-1) != 1:
            raise L.B200Error(L.ERR_INVALID, f"gemm: {nm} must have a contiguous last dimension")
    p.m, p.n, p.k = m, n, k
    p.batch_outer = p.batch_inner = 1
    p.lda, p.ldb, p.ldc = a.stride(0), b.stride(0), out.stride(0)
    p.epilogue = act | (L.EPI_BIAS if bias is not None else 0) | (L.EPI_RESIDUAL if residual is not None else 0)
    p.alpha, p.bias_scale, p.residual_scale = alpha, bias_scale, residual_scale
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    if residual is not None:
        p.residual, p.ldr = residual.data_ptr(), residual.stride(0)
    if ln is not None:
        p.epilogue |= L.EPI_LAYERNORM
        p.ln_gamma = ln[0].data_ptr() if ln[0] is not None else None
        p.ln_beta = ln[1].data_ptr() if ln[1] is not None else None
        p.ln_eps = ln[2]
    gemm_raw(ctx, p, _stream(a))
    return out


def gemm_batched(a, b, out, *, b_layout=0, alpha=1.0, bias=None, act=0):
    """Batched product over two leading batch axes given as 4-D strided views [B1, B2, rows, cols]
    (last dimension contiguous; a batch stride of 0 broadcasts)."""
    ctx = _ctx(a)
    p = L.GemmParams()
    p.dtype = L.dtype_code(a.dtype)
    p.a_layout, p.b_layout = 0, b_layout
    b1, b2, m, k = a.shape
    n = b.shape[3] if b_layout == 0 else b.shape[2]
    p.m, p.n, p.k = m, n, k
    p.batch_outer, p.batch_inner = b1, b2
    p.lda, p.a_stride_outer, p.a_stride_inner = a.stride(2), a.stride(0), a.stride(1)
    p.ldb, p.b_stride_outer, p.b_stride_inner = b.stride(2), b.stride(0), b.stride(1)
    p.ldc, p.c_stride_outer, p.c_stride_inner = out.stride(2), out.stride(0), out.stride(1)
    p.epilogue = act | (L.EPI_BIAS if bias is not None else 0)
    p.alpha, p.bias_scale, p.residual_scale = alpha, 1.0, 1.0
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), out.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    gemm_raw(ctx, p, _stream(a))
    return out


def softmax(x, out, *, rows, cols, scale=1.0, mask=None, mask_row_div=1, log=False):
    ctx = _ctx(x)
    _contig(x, "softmax input"), _contig(out, "softmax output"), _contig(mask, "softmax mask")
    L.check(ctx.lib.b200ml_softmax(ctx.handle, L.dtype_code(x.dtype), L.ptr(x), L.ptr(mask), L.ptr(out), rows, cols,
                                   mask_row_div, scale, 1 if log else 0, _stream(x)))
    return out


def layernorm(x, out, *, gamma=None, beta=None, residual=None, bias=None, eps=1e-5):
    ctx = _ctx(x)
    for t in (x, out, gamma, beta, residual, bias):
        _contig(t, "layernorm operand")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    L.check(ctx.lib.b200ml_layernorm(ctx.handle, L.dtype_code(x.dtype), L.ptr(x), L.ptr(residual), L.ptr(bias),
                                     L.ptr(gamma), L.ptr(beta), L.ptr(out), rows, cols, eps, _stream(x)))
    return out


def reduce(x, out, *, op, outer, red, inner):
    ctx = _ctx(x)
    _contig(x, "reduce input"), _contig(out, "reduce output")
    L.check(ctx.lib.b200ml_reduce(ctx.handle, L.dtype_code(x.dtype), op, L.ptr(x), L.ptr(out), outer, red, inner,
                                  _stream(x)))
    return out


def unary(x, out, op, p0=0.0, p1=0.0):
    ctx = _ctx(x)
    _contig(x, "unary input"), _contig(out, "unary output")
    L.check(ctx.lib.b200ml_unary(ctx.handle, L.dtype_code(x.dtype), op, L.ptr(x), L.ptr(out), x.numel(), p0, p1,
                                 _stream(x)))
    return out


def binary(a, b, out, op):
    """Numpy-broadcast ``out = a <op> b``; operands are expanded to the output shape by strides."""
    ctx = _ctx(out)
    _contig(out, "binary output")
    shape = list(out.shape)
    if len(shape) > 6:
        raise L.Unsupported(L.ERR_UNSUPPORTED, "binary: rank > 6")
    ae, be = a.expand(shape), b.expand(shape)
    L.check(ctx.lib.b200ml_binary(ctx.handle, L.dtype_code(out.dtype), op, L.ptr(a), L.ptr(b), L.ptr(out), len(shape),
                                  _i64(shape), _i64(ae.stride()), _i64(be.stride()), _stream(out)))
    return out


def bias_act(x, out, *, bias=None, residual=None, act=0):
    ctx = _ctx(x)
    for t in (x, out, bias, residual):
        _contig(t, "bias_act operand")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    L.check(ctx.lib.b200ml_bias_act(ctx.handle, L.dtype_code(x.dtype), L.ptr(x), L.ptr(bias), L.ptr(residual),
                                    L.ptr(out), rows, cols, act, _stream(x)))
    return out


def transpose(x, out, perm):
    ctx = _ctx(x)
    _contig(x, "transpose input"), _contig(out, "transpose output")
    if x.element_size() not in (2, 4):
        raise L.Unsupported(L.ERR_UNSUPPORTED, f"transpose: element size {x.element_size()}")
    if x.dim() > 6:
        raise L.Unsupported(L.ERR_UNSUPPORTED, "transpose: rank > 6")
    L.check(ctx.lib.b200ml_transpose(ctx.handle, x.element_size(), L.ptr(x), L.ptr(out), x.dim(), _i64(x.shape),
                                     _i32(perm), _stream(x)))
    return out


def cast(x, out):
    ctx = _ctx(x)
    _contig(x, "cast input"), _contig(out, "cast output")
    L.check(ctx.lib.b200ml_cast(ctx.handle, L.cast_code(x.dtype), L.cast_code(out.dtype), L.ptr(x), L.ptr(out),
                                x.numel(), _stream(x)))
    return out


def strided_copy(src, dst):
    """``dst[...] = src`` for two views of the same shape (torch views carry offset and strides: ``narrow`` gives the
    sub-ranges of Slice / Split / Concat, ``expand`` the stride-0 axes of Expand)."""
    ctx = _ctx(dst)
    if tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype:
        raise L.B200Error(L.ERR_INVALID, f"strided_copy: {tuple(src.shape)} {src.dtype} into {tuple(dst.shape)} {dst.dtype}")
    if src.dim() > 6:
        raise L.Unsupported(L.ERR_UNSUPPORTED, "strided_copy: rank > 6")
    if src.numel() == 0:
        return dst
    L.check(ctx.lib.b200ml_strided_copy(ctx.handle, src.element_size(), L.ptr(src), L.ptr(dst), src.dim(), _i64(src.shape),
                                        _i64(src.stride()), _i64(dst.stride()), _stream(dst)))
    return dst


def strided_copy_parts(srcs, dsts):
    """``dsts[i][...] = srcs[i]`` for several pairs of equally shaped views of one dtype and rank: the parts of a Split
    or a Concat in one launch (eight parts per launch)."""
    if len(srcs) != len(dsts) or not srcs:
        raise L.B200Error(L.ERR_INVALID, "strided_copy_parts: need as many sources as destinations, at least one")
    rank, dtype = srcs[0].dim(), srcs[0].dtype
    pairs = [(s_, d_) for s_, d_ in zip(srcs, dsts) if s_.numel() > 0]
    for s_, d_ in zip(srcs, dsts):
        if tuple(s_.shape) != tuple(d_.shape) or s_.dtype != dtype or d_.dtype != dtype or s_.dim() != rank:
            raise L.B200Error(L.ERR_INVALID, "strided_copy_parts: parts must agree in dtype and rank, and each pair in shape")
    if rank == 0 or rank > 6 or len(pairs) == 1:
        for s_, d_ in pairs:
            strided_copy(s_, d_)
        return dsts
    ctx = _ctx(dsts[0])
    for lo in range(0, len(pairs), 8):
        chunk = pairs[lo:lo + 8]
        n = len(chunk)
        xs = (ctypes.c_void_p * n)(*[s_.data_ptr() for s_, _ in chunk])
        ys = (ctypes.c_void_p * n)(*[d_.data_ptr() for _, d_ in chunk])
        shapes = _i64([e for s_, _ in chunk for e in s_.shape])
        xst = _i64([e for s_, _ in chunk for e in s_.stride()])
        yst = _i64([e for _, d_ in chunk for e in d_.stride()])
        L.check(ctx.lib.b200ml_strided_copy_parts(ctx.handle, dtype.itemsize, n, xs, ys, rank, shapes, xst, yst, _stream(dsts[0])))
    return dsts


def gather(data, indices, out, axis=0):
    """``out = numpy.take(data, indices, axis)`` with int64 ``indices`` of any shape."""
    ctx = _ctx(data)
    for t in (data, indices, out):
        _contig(t, "gather operand")
    if indices.dtype != torch.int64:
        raise L.B200Error(L.ERR_INVALID, f"gather: indices must be int64, got {indices.dtype}")
    axis %= max(data.dim(), 1)
    outer = 1
    for d in data.shape[:axis]:
        outer *= d
    inner = 1
    for d in data.shape[axis + 1:]:
        inner *= d
    if tuple(out.shape) != tuple(data.shape[:axis]) + tuple(indices.shape) + tuple(data.shape[axis + 1:]) or out.dtype != data.dtype:
        raise L.B200Error(L.ERR_INVALID, f"gather: output is {tuple(out.shape)} {out.dtype}")
    L.check(ctx.lib.b200ml_gather(ctx.handle, data.element_size(), L.ptr(data), L.ptr(indices), L.ptr(out), outer,
                                  data.shape[axis], inner, indices.numel(), _stream(data)))
    return out


def where(condition, x, y, out):
    """Numpy-broadcast ``out = condition ? x : y``; ``condition`` is a bool (or uint8) tensor."""
    ctx = _ctx(out)
    _contig(out, "where output")
    if condition.dtype not in (torch.bool, torch.uint8) or x.dtype != out.dtype or y.dtype != out.dtype:
        raise L.B200Error(L.ERR_INVALID, f"where: dtypes {condition.dtype}, {x.dtype}, {y.dtype} -> {out.dtype}")
    shape = list(out.shape)
    if len(shape) > 6 or out.element_size() not in (2, 4, 8):
        raise L.Unsupported(L.ERR_UNSUPPORTED, "where: rank > 6 or element size not 2 / 4 / 8")
    ce, xe, ye = condition.expand(shape), x.expand(shape), y.expand(shape)
    L.check(ctx.lib.b200ml_where(ctx.handle, out.element_size(), L.ptr(condition), L.ptr(x), L.ptr(y), L.ptr(out), len(shape),
                                 _i64(shape), _i64(ce.stride()), _i64(xe.stride()), _i64(ye.stride()), _stream(out)))
    return out


def compare(a, b, out, op):
    """Numpy-broadcast ``out = a <op> b`` into a bool (or uint8) tensor; operands are float16, float32 or int64."""
    ctx = _ctx(out)
    _contig(out, "compare output")
    if a.dtype != b.dtype or out.dtype not in (torch.bool, torch.uint8):
        raise L.B200Error(L.ERR_INVALID, f"compare: dtypes {a.dtype}, {b.dtype} -> {out.dtype}")
    code = L.I64 if a.dtype == torch.int64 else L.dtype_code(a.dtype)
    shape = list(out.shape)
    if len(shape) > 6:
        raise L.Unsupported(L.ERR_UNSUPPORTED, "compare: rank > 6")
    ae, be = a.expand(shape), b.expand(shape)
    L.check(ctx.lib.b200ml_compare(ctx.handle, code, op, L.ptr(a), L.ptr(b), L.ptr(out), len(shape), _i64(shape),
                                   _i64(ae.stride()), _i64(be.stride()), _stream(out)))
    return out


def maxpool2d(x, out, *, kernel, strides=(1, 1), pads=(0, 0, 0, 0)):
    """NCHW max pooling, floor mode; ``pads`` is ONNX order (top, left, bottom, right)."""
    ctx = _ctx(x)
    _contig(x, "maxpool input"), _contig(out, "maxpool output")
    n, c, h, w = x.shape
    oh = (h + pads[0] + pads[2] - kernel[0]) // strides[0] + 1
    ow = (w + pads[1] + pads[3] - kernel[1]) // strides[1] + 1
    if tuple(out.shape) != (n, c, oh, ow):
        raise L.B200Error(L.ERR_INVALID, f"maxpool2d: output is {tuple(out.shape)}, expected {(n, c, oh, ow)}")
    L.check(ctx.lib.b200ml_maxpool2d(ctx.handle, L.dtype_code(x.dtype), L.ptr(x), L.ptr(out), n * c, h, w, kernel[0], kernel[1],
                                     strides[0], strides[1], pads[0], pads[1], pads[2], pads[3], _stream(x)))
    return out


def _conv_params(x_shape, dtype, w, bias, strides, pads, dilations, group, act):
    p = L.ConvParams()
    p.dtype, p.act = L.dtype_code(dtype), act
    p.n, p.c, p.h, p.w = x_shape
    p.m, _, p.kh, p.kw = w.shape
    p.stride_h, p.stride_w = strides
    p.pad_top, p.pad_left, p.pad_bottom, p.pad_right = pads
    p.dil_h, p.dil_w = dilations
    p.group = group
    p.weight = w.data_ptr()
    p.bias = bias.data_ptr() if bias is not None else None
    return p


def conv2d(x, w, out, *, bias=None, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1, act=0, gate=None,
           residual=None, pool_mean=None, packed_weight=None):
    """ONNX Conv on NCHW tensors; ``pads`` is ONNX order (top, left, bottom, right).  ``packed_weight``: what
    :func:`conv_prepack` returned for these weights, bias, shapes and attributes (or None)."""
    ctx = _ctx(x)
    for t in (x, w, out, bias, gate, residual, pool_mean):
        _contig(t, "conv operand")
    p = _conv_params(x.shape, x.dtype, w, bias, strides, pads, dilations, group, act)
    p.x, p.y = x.data_ptr(), out.data_ptr()
    p.gate = gate.data_ptr() if gate is not None else None
    p.residual = residual.data_ptr() if residual is not None else None
    p.pool_sum = pool_mean.data_ptr() if pool_mean is not None else None
    p.packed_weight = packed_weight.data_ptr() if packed_weight is not None else None
    L.check(ctx.lib.b200ml_conv2d(ctx.handle, ctypes.byref(p), _stream(x)))
    return out


def conv_prepack(x_shape, w, *, bias=None, strides=(1, 1), pads=(0, 0, 0, 0), dilations=(1, 1), group=1, gate=False):
    """Prepares constant convolution weights once (``b200ml_conv_prepack``): returns the packed tensor to pass to
    :func:`conv2d` as ``packed_weight``, or None when this convolution runs on a kernel that takes the weights as they
    are.  ``w`` and ``bias`` are device tensors; ``gate`` says whether the calls will carry a squeeze-excite gate."""
    if not w.is_cuda or w.dtype != torch.float32:
        return None
    ctx = _ctx(w)
    for t in (w, bias):
        _contig(t, "conv operand")
    p = _conv_params(x_shape, w.dtype, w, bias, strides, pads, dilations, group, 0)
    p.gate = 1 if gate else None  # only its presence matters (the implicit-GEMM kernel takes no gate)
    nbytes = int(ctx.lib.b200ml_conv_prepack_bytes(ctx.handle, ctypes.byref(p)))
    if nbytes <= 0:
        return None
    packed = torch.empty(nbytes, dtype=torch.uint8, device=w.device)
    L.check(ctx.lib.b200ml_conv_prepack(ctx.handle, ctypes.byref(p), ctypes.c_void_p(packed.data_ptr()), _stream(w)))
    return packed


def se_gate(pooled, w1, b1, w2, b2, out):
    ctx = _ctx(pooled)
    for t in (pooled, w1, b1, w2, b2, out):
        _contig(t, "se_gate operand")
    n = pooled.shape[0]
    c = pooled.numel() // n if n else 0
    r = w1.shape[0]
    L.check(ctx.lib.b200ml_se_gate(ctx.handle, L.dtype_code(pooled.dtype), L.ptr(pooled), L.ptr(w1), L.ptr(b1),
                                   L.ptr(w2), L.ptr(b2), L.ptr(out), n, c, r, _stream(pooled)))
    return out


def attention(q, k, v, out, *, scale, mask=None):
    """Fused softmax(scale * Q K^T + mask) V on 4-D strided views [B, heads, S, head_dim] (fp16)."""
    ctx = _ctx(q)
    p = L.AttentionParams()
    p.batch, p.heads, p.seq_q, p.head_dim = q.shape
    p.seq_kv = k.shape[2]
    for t, nm in ((q, "q"), (k, "k"), (v, "v"), (out, "o")):
        if t.stride(3) != 1:
            raise L.B200Error(L.ERR_INVALID, f"attention: {nm} must have a contiguous head dimension")
        if t.dtype != torch.float16:
            raise L.Unsupported(L.ERR_UNSUPPORTED, "attention: float16 only")
    p.q_stride_b, p.q_stride_h, p.q_stride_s = q.stride(0), q.stride(1), q.stride(2)
    p.k_stride_b, p.k_stride_h, p.k_stride_s = k.stride(0), k.stride(1), k.stride(2)
    p.v_stride_b, p.v_stride_h, p.v_stride_s = v.stride(0), v.stride(1), v.stride(2)
    p.o_stride_b, p.o_stride_h, p.o_stride_s = out.stride(0), out.stride(1), out.stride(2)
    p.scale = scale
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    if mask is not None and (mask.dtype != torch.float16 or mask.numel() != p.batch * p.seq_kv or not mask.is_contiguous()):
        raise L.B200Error(L.ERR_INVALID, "attention: the additive mask must be %d x %d contiguous float16 values, got %s %s"
                          % (p.batch, p.seq_kv, tuple(mask.shape), mask.dtype))
    p.mask = mask.data_ptr() if mask is not None else None
    L.check(ctx.lib.b200ml_attention_f16(ctx.handle, ctypes.byref(p), _stream(q)))
    return out
