"""Data-movement operators on the B200 (Slice, Split, Concat, Expand, Gather, Where, MaxPool, Shape): bit-exact against
the CPU oracle, on the reference's own test cases (tests/pure_expansions/test_expansions.py:464-563), ragged and
unaligned shapes, every element size, and at sizes above the L2 through round-trip properties."""
import numpy as np
import pytest
import torch

import daceml_b200.onnx as donnx
from daceml_b200 import kernels as K, lib as L
from daceml_b200.onnx.exported_graph import ExportedGraph, GraphNode, ValueInfo
from daceml_b200.onnx.onnx_importer import ONNXModel
from oracle import ops

pytestmark = pytest.mark.gpu
NP = {torch.float32: np.float32, torch.float16: np.float16, torch.int64: np.int64, torch.uint8: np.uint8, torch.float64: np.float64}
I64MAX = (1 << 63) - 1


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def empty(shape, dtype):
    return torch.empty(tuple(shape), dtype=dtype, device="cuda")


def data(rng, shape, dtype):
    if dtype in (torch.int64, torch.uint8):
        return rng.integers(0, 200, shape).astype(NP[dtype])
    return rng.standard_normal(shape).astype(NP[dtype])


def status_ok():
    torch.cuda.synchronize()
    assert L.get_context(0).device_status() == 0


def same(t, ref):
    got = t.cpu().numpy()
    assert got.shape == ref.shape and got.dtype == ref.dtype, (got.shape, got.dtype, ref.shape, ref.dtype)
    assert np.array_equal(got, ref)


# ------------------------------------------------------------------------------------------------
# Gather / Shape: the reference's tests
# ------------------------------------------------------------------------------------------------
def test_shape_reference_test():
    inp = dev(np.random.rand(9, 5, 3))
    shp = empty((3, ), torch.int64)
    donnx.ONNXShape(data=inp, shape=shp)
    assert shp.tolist() == [9, 5, 3]


def test_gather_reference_tests(rng):
    d = np.array([[1.0, 1.2], [2.3, 3.4], [4.5, 5.7]])
    idx = np.array([[0, 1], [1, 2]])
    out = empty((2, 2, 2), torch.float64)
    donnx.ONNXGather(data=dev(d), output=out, indices=dev(idx), axis=0)
    same(out, d[idx])
    same(out, ops.gather(d, idx, 0))
    embs, ids = rng.random((64, 8)), rng.integers(0, 64, (8, 16))  # the lookup at the start of a BERT model
    out = empty((8, 16, 8), torch.float64)
    donnx.ONNXGather(data=dev(embs), output=out, indices=dev(ids), axis=0)
    same(out, embs[ids])
    d3 = rng.random((1, 8, 32))  # scalar index, third last operator of a BERT model
    out = empty((1, 32), torch.float64)
    donnx.ONNXGather(data=dev(d3), output=out, indices=torch.tensor(5).cuda(), axis=1)
    same(out, np.take(d3, 5, axis=1))
    d2 = np.array([[1.0, 1.2, 1.9], [2.3, 3.4, 3.9], [4.5, 5.7, 5.9]])
    out = empty((3, 1, 2), torch.float64)
    donnx.ONNXGather(data=dev(d2), output=out, indices=dev(np.array([[0, 2]])), axis=1)
    same(out, np.take(d2, np.array([[0, 2]]), axis=1))
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64, torch.uint8])
@pytest.mark.parametrize("shape, axis, ishape", [((1000, 1024), 0, (8, 512)), ((7, 33, 5), 1, (4, )), ((5, 6, 7), 2, (2, 3)),
                                                 ((30522, 127), 0, (3, 129)), ((6, ), 0, (11, ))])
def test_gather_shapes_and_negative_indices(dtype, shape, axis, ishape, rng):
    d = data(rng, shape, dtype)
    idx = rng.integers(-shape[axis], shape[axis], ishape)
    ref = ops.gather(d, idx, axis)
    out = empty(ref.shape, dtype)
    K.gather(dev(d), dev(idx), out, axis)
    same(out, ref)
    status_ok()


def test_gather_bad_index_sets_status_and_writes_zero(rng):
    d = data(rng, (10, 8), torch.float32)
    idx = np.array([0, 10, 3, -11])
    out = empty((4, 8), torch.float32)
    K.gather(dev(d), dev(idx), out, 0)
    torch.cuda.synchronize()
    with pytest.raises(L.B200Error, match="index outside"):
        L.get_context(0).device_status()
    got = out.cpu().numpy()
    assert np.array_equal(got[0], d[0]) and np.array_equal(got[2], d[3]) and not got[1].any() and not got[3].any()
    assert L.get_context(0).device_status() == 0  # reading the status clears it


# ------------------------------------------------------------------------------------------------
# Slice / Split / Concat / Expand
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64, torch.uint8])
@pytest.mark.parametrize("shape, starts, ends, axes, steps", [
    ((20, 16), [2], [I64MAX], [0], [1]),                      # the reference's form: axis 0, step 1, exporter's "to the end"
    ((8, 512, 1024), [0], [1], [1], [1]),                     # the [CLS] row of every sequence
    ((4, 33, 65), [1, -40], [30, 1000], [1, 2], [3, 2]),      # steps, negative start, clamped end
    ((6, 7, 8, 9), [1, 2, 3], [5, 6, 7], None, None),         # axes and steps omitted
    ((3, 40), [8], [24], [-1], [1]),                          # aligned inner sub-range: the 16-byte path
    ((5, 5), [3], [2], [0], [1]),                             # empty result
])
def test_slice_against_oracle(dtype, shape, starts, ends, axes, steps, rng):
    d = data(rng, shape, dtype)
    ref = ops.slice_(d, starts, ends, axes, steps)
    out = empty(ref.shape, dtype)
    kwargs = dict(data=dev(d), output=out, starts=np.array(starts), ends=np.array(ends))
    if axes is not None:
        kwargs.update(axes=np.array(axes), steps=np.array(steps))
    donnx.ONNXSlice(**kwargs)
    same(out, ref)
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape, axis, sizes", [((8, 512, 3072), 2, [1024, 1024, 1024]), ((9, 7), 0, [2, 3, 4]), ((4, 10, 6), 1, None)])
def test_split_and_concat_round_trip(dtype, shape, axis, sizes, rng):
    d = data(rng, shape, dtype)
    parts = ops.split(d, axis, sizes, parts=2)
    outs = [empty(p.shape, dtype) for p in parts]
    kwargs = {"outputs__%d" % i: o for i, o in enumerate(outs)}
    if sizes is not None:
        kwargs["split"] = sizes
    donnx.ONNXSplit(input=dev(d), axis=axis, **kwargs)
    for o, p in zip(outs, parts):
        same(o, p)
    back = empty(shape, dtype)
    donnx.ONNXConcat(concat_result=back, axis=axis, **{"inputs__%d" % i: o for i, o in enumerate(outs)})
    same(back, d)
    same(back, ops.concat(parts, axis))
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("shape, target", [((3, 1), (2, 3, 4)), ((1, 1, 512), (8, 512, 512)), ((5, 4), (5, 4)), ((1, ), (7, )), ((2, 1, 6), (2, 5, 6))])
def test_expand_broadcasts(dtype, shape, target, rng):
    d = data(rng, shape, dtype)
    ref = ops.expand(d, target)
    out = empty(ref.shape, dtype)
    donnx.ONNXExpand(input=dev(d), shape=np.array(target), output=out)
    same(out, ref)
    status_ok()


def test_strided_copy_rejects_bad_arguments():
    a, b = empty((4, 4), torch.float32), empty((4, 5), torch.float32)
    with pytest.raises(L.B200Error):
        K.strided_copy(a, b)
    with pytest.raises(L.B200Error):
        K.strided_copy(a.expand(2, 4, 4), empty((4, 4), torch.float32).expand(2, 4, 4))  # destination broadcast
    K.strided_copy(empty((0, 4), torch.float32), empty((0, 4), torch.float32))  # nothing to do
    status_ok()


def test_large_slice_and_gather_properties(rng):
    """Above the L2: slicing the two halves of a 256 MB tensor and concatenating them gives the tensor back; gathering
    with a permutation and then with its inverse is the identity."""
    x = torch.randn(8192, 8192, device="cuda")
    lo, hi = empty((8192, 4096), torch.float32), empty((8192, 4096), torch.float32)
    donnx.ONNXSlice(data=x, output=lo, starts=np.array([0]), ends=np.array([4096]), axes=np.array([1]), steps=np.array([1]))
    donnx.ONNXSlice(data=x, output=hi, starts=np.array([4096]), ends=np.array([I64MAX]), axes=np.array([1]), steps=np.array([1]))
    back = torch.empty_like(x)
    donnx.ONNXConcat(concat_result=back, axis=1, inputs__0=lo, inputs__1=hi)
    assert torch.equal(back, x)
    perm = torch.randperm(8192, device="cuda")
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(8192, device="cuda")
    g1, g2 = torch.empty_like(x), torch.empty_like(x)
    K.gather(x, perm, g1, 0)
    K.gather(g1, inv, g2, 0)
    assert torch.equal(g2, x) and not torch.equal(g1, x)
    status_ok()


# ------------------------------------------------------------------------------------------------
# Where / MaxPool
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64])
@pytest.mark.parametrize("cshape, xshape, yshape", [((4, 5), (4, 5), (4, 5)), ((8, 1, 1, 128), (8, 4, 128, 128), ()), ((3, 1), (1, 7), (3, 7)),
                                                    ((1000, 1001), (1000, 1001), (1, ))])
def test_where_broadcasts(dtype, cshape, xshape, yshape, rng):
    c = rng.integers(0, 2, cshape).astype(bool)
    x, y = data(rng, xshape, dtype), data(rng, yshape, dtype)
    ref = ops.where(c, x, y)
    out = empty(ref.shape, dtype)
    donnx.ONNXWhere(condition=dev(c), X=dev(x), Y=dev(y), output=out)
    same(out, ref)
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64])
def test_comparisons(dtype, rng):
    a, b = data(rng, (33, 65), dtype), data(rng, (65, ), dtype)
    b[:9] = a[7, :9]  # some equal pairs
    if dtype != torch.int64:
        a[3, 3] = np.nan  # NaN compares false
    for name, fn in (("Equal", np.equal), ("Greater", np.greater), ("Less", np.less), ("GreaterOrEqual", np.greater_equal),
                     ("LessOrEqual", np.less_equal)):
        out = empty((33, 65), torch.bool)
        getattr(donnx, "ONNX" + name)(A=dev(a), B=dev(b), C=out)
        same(out, fn(a, b))
        # the vectorised forms: a full second operand, and a scalar one
        full = np.ascontiguousarray(np.broadcast_to(b, a.shape))
        getattr(donnx, "ONNX" + name)(A=dev(a), B=dev(full), C=out)
        same(out, fn(a, full))
        getattr(donnx, "ONNX" + name)(A=dev(a), B=dev(b[4:5].reshape(())), C=out)
        same(out, fn(a, b[4]))
    status_ok()


CAST_TYPES = [torch.float16, torch.float32, torch.float64, torch.int32, torch.int64, torch.uint8, torch.bool]


@pytest.mark.parametrize("src", CAST_TYPES)
def test_cast_between_all_types(src, rng):
    """tests/pure_expansions/test_expansions.py:85-184 (int -> float, float -> int, float -> long), widened to every
    pair: values are small enough for every target, floats carry fractions so that truncation toward zero shows."""
    if src == torch.bool:
        x = rng.integers(0, 2, (37, 65)).astype(bool)
    elif src.is_floating_point:
        x = (rng.standard_normal((37, 65)) * 20).clip(0.0, 100.0).astype(NP[src])
        x[0, :4] = [0.0, 0.4, 0.99, 1.5]
    else:
        x = rng.integers(0, 100, (37, 65)).astype({torch.int32: np.int32}.get(src, NP.get(src)))
    for dst in CAST_TYPES:
        np_dst = {torch.int32: np.int32, torch.bool: bool}.get(dst, NP.get(dst))
        out = empty(x.shape, dst)
        donnx.ONNXCast(input=dev(x), output=out, to=1)
        same(out, x.astype(np_dst))
    status_ok()


def test_cast_negative_floats_truncate_toward_zero():
    x = np.array([-2.7, -0.5, 0.5, 2.7, -100.9], dtype=np.float32)
    out = empty(x.shape, torch.int64)
    donnx.ONNXCast(input=dev(x), output=out, to=7)
    assert out.tolist() == [-2, 0, 0, 2, -100]


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape, kernel, strides, pads", [((2, 6, 28, 28), (2, 2), (2, 2), (0, 0, 0, 0)),   # LeNet pooling
                                                           ((3, 5, 17, 23), (3, 3), (2, 2), (1, 1, 1, 1)),   # ResNet stem form, ragged
                                                           ((1, 4, 9, 9), (3, 2), (1, 3), (2, 0, 0, 1)),     # asymmetric pads
                                                           ((2, 3, 8, 8), (8, 8), (1, 1), (0, 0, 0, 0))])    # one window per plane
def test_maxpool_against_oracle_and_torch(dtype, shape, kernel, strides, pads, rng):
    x = data(rng, shape, dtype)
    ref = ops.maxpool2d(x, kernel, strides, pads)
    out = empty(ref.shape, dtype)
    donnx.ONNXMaxPool(X=dev(x), Y=out, kernel_shape=list(kernel), strides=list(strides), pads=list(pads))
    same(out, ref)
    if pads[0] == pads[2] and pads[1] == pads[3]:
        t = torch.nn.functional.max_pool2d(torch.from_numpy(x).float(), kernel, strides, padding=(pads[0], pads[1]))
        assert np.array_equal(out.float().cpu().numpy(), t.numpy())
    status_ok()


def test_maxpool_rejects_what_it_cannot_do():
    x, y = empty((1, 1, 8, 8), torch.float32), empty((1, 1, 4, 4), torch.float32)
    with pytest.raises(NotImplementedError):
        donnx.ONNXMaxPool(X=x, Y=y, kernel_shape=[2, 2], strides=[2, 2], ceil_mode=1)
    with pytest.raises(NotImplementedError):
        donnx.ONNXMaxPool(X=x, Y=y, kernel_shape=[2, 2], strides=[2, 2], dilations=[2, 2])
    with pytest.raises(L.B200Error):
        K.maxpool2d(x, empty((1, 1, 6, 6), torch.float32), kernel=(2, 2), strides=(2, 2), pads=(2, 2, 2, 2))


# ------------------------------------------------------------------------------------------------
# through the importer: an embedding front end (Gather + Add + Slice + Concat) as an exported graph
# ------------------------------------------------------------------------------------------------
def test_embedding_graph_through_importer(rng):
    class Front(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tok, self.pos = torch.nn.Embedding(1000, 64), torch.nn.Embedding(32, 64)

        def forward(self, ids):
            h = self.tok(ids) + self.pos.weight[:ids.shape[1]]
            return torch.cat([h[:, :1], h[:, -1:]], dim=1), torch.where(h > 0, h, torch.zeros_like(h))

    torch.manual_seed(0)
    net = Front()
    ids = torch.from_numpy(rng.integers(0, 1000, (4, 16)))
    model = ONNXModel.from_torch("front", net, (ids, ))
    got = model(ids.cuda())
    with torch.no_grad():
        ref = net(ids)
    for g, r in zip(got, ref):
        assert torch.equal(g.cpu(), r)
    status_ok()


def test_tiny_bert_with_mask_through_dace_module(rng):
    """Embeddings (Gather), position slice, LayerNorm, the run-time attention mask ((1 - mask) * -10000 broadcast over
    heads and queries), two HF encoder layers, [CLS] Gather and the Tanh pooler, from one ``nn.Module``."""
    import copy
    from daceml_b200.torch import DaceModule
    from conftest import assert_close
    from models import TinyBert
    net = TinyBert().half().eval()
    ref_net = copy.deepcopy(net).float()
    ids = torch.from_numpy(rng.integers(0, 1000, (4, 64)))
    mask = torch.ones(4, 64, dtype=torch.int64)
    mask[1, 40:] = 0
    mask[3, 7:] = 0
    module = DaceModule(net.cuda())
    hidden, pooled = module(ids.cuda(), mask.cuda())
    names = module.compiled_function.kernel_names()
    assert names.count("attention") == 2 and names.count("gather") == 2 and "cast" in names
    with torch.no_grad():
        ref_hidden, ref_pooled = ref_net(ids, mask)
    assert_close(hidden, ref_hidden, dtype=torch.float16, what="hidden states")
    assert_close(pooled, ref_pooled, dtype=torch.float16, what="pooled output")
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.int64, torch.bool])
def test_strided_copy_parts_is_one_launch_per_eight_parts(dtype, rng):
    """Split and Concat through the multi-part copy: all parts in one launch when they move the same unit, parts of
    odd widths (different units) and more than eight parts included; bit-exact against torch slicing."""
    def make(*shape):
        if dtype == torch.bool:
            return torch.from_numpy(rng.random(shape) > 0.5).cuda()
        if dtype == torch.int64:
            return torch.from_numpy(rng.integers(-1000, 1000, shape)).cuda()
        return torch.from_numpy(rng.standard_normal(shape).astype(np.float32)).to(dtype).cuda()

    x = make(37, 3 * 64)
    parts = [torch.empty(37, 64, dtype=dtype, device="cuda") for _ in range(3)]
    before = L.launch_count()
    K.strided_copy_parts([x.narrow(1, 64 * j, 64) for j in range(3)], parts)
    assert L.launch_count() - before == 1
    for j in range(3):
        assert torch.equal(parts[j], x[:, 64 * j:64 * (j + 1)])
    # Concat of ragged widths (7, 64, 9 columns: not all 16-byte units) into one row-major output
    widths = [7, 64, 9]
    srcs = [make(11, w) for w in widths]
    out = torch.zeros(11, sum(widths), dtype=dtype, device="cuda")
    off, dsts = 0, []
    for w in widths:
        dsts.append(out.narrow(1, off, w))
        off += w
    K.strided_copy_parts(srcs, dsts)
    assert torch.equal(out, torch.cat(srcs, dim=1))
    # eleven parts along axis 0: two launches
    big = make(11 * 5, 24)
    outs = [torch.empty(5, 24, dtype=dtype, device="cuda") for _ in range(11)]
    before = L.launch_count()
    K.strided_copy_parts([big.narrow(0, 5 * j, 5) for j in range(11)], outs)
    assert L.launch_count() - before == 2
    for j in range(11):
        assert torch.equal(outs[j], big[5 * j:5 * j + 5])
    torch.cuda.synchronize()
    assert L.get_context(0).device_status() == 0
