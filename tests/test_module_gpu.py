"""``DaceModule`` / ``ONNXModel`` on the B200: real ``nn.Module`` objects in, results against PyTorch.

The reference's tests of the same shape are ``tests/torch/test_bert_encoder.py:11-33`` (HF BertLayer against
PyTorch), ``tests/torch/test_conv2d.py:14-42`` and the README network; tolerances are the configured ones
(rtol 1e-4 fp32, 2e-2 fp16)."""
import copy
import warnings

import pytest
import torch
import torch.nn as nn

from daceml_b200 import lib as L
from daceml_b200.onnx.onnx_importer import ONNXModel
from daceml_b200.torch import DaceModule, dace_module
from conftest import assert_close
from models import LeNet, MLP, MBConv, bert_layer

pytestmark = pytest.mark.gpu
warnings.filterwarnings("ignore")


def status_ok():
    torch.cuda.synchronize()
    assert L.get_context(0).device_status() == 0


@pytest.mark.parametrize("cuda_graph", [False, True])
def test_hf_bert_layer_through_dace_module(cuda_graph):
    layer = bert_layer(256, 4, 512).half()
    ref_layer = copy.deepcopy(layer).float()  # fp32 arithmetic on the fp16-rounded weights
    torch.manual_seed(1)
    x = torch.randn(2, 128, 256).half()
    module = DaceModule(layer.cuda(), cuda_graph=cuda_graph)
    y = module(x.cuda())
    assert module.compiled_function.kernel_names() == ["gemm", "attention", "gemm_layernorm", "gemm", "gemm_layernorm"]
    with torch.no_grad():
        ref = ref_layer(x.float())
    ref = ref[0] if isinstance(ref, tuple) else ref
    assert y.dtype == torch.float16 and y.is_cuda
    assert_close(y, ref, dtype=torch.float16, what="BertLayer")
    # a second call with other data reuses the compiled plan
    x2 = torch.randn(2, 128, 256).half()
    y2 = module(x2.cuda())
    with torch.no_grad():
        ref2 = ref_layer(x2.float())
    ref2 = ref2[0] if isinstance(ref2, tuple) else ref2
    assert_close(y2, ref2, dtype=torch.float16, what="BertLayer, second call")
    status_ok()


def test_bert_large_layer_full_size_through_dace_module():
    """The benchmark layer (1024 / 16 / 4096, batch 8, sequence 512) from the HF module: same launches as the
    hand-built runner, result against PyTorch's fp16 CUDA layer within the fp16 tolerance."""
    layer = bert_layer(1024, 16, 4096).half().cuda()
    torch.manual_seed(2)
    x = torch.randn(8, 512, 1024).half().cuda()
    module = DaceModule(layer, cuda_graph=True)
    y = module(x)
    assert module.compiled_function.kernel_names() == ["gemm", "attention", "gemm_layernorm", "gemm", "gemm_layernorm"]
    with torch.no_grad():
        ref = layer.float()(x.float())
    ref = ref[0] if isinstance(ref, tuple) else ref
    assert_close(y, ref, dtype=torch.float16, what="BERT-large layer")
    status_ok()


def test_mlp_module_matches_pytorch():
    torch.manual_seed(0)
    net = MLP()
    x = torch.randn(4096, 784)
    module = DaceModule(copy.deepcopy(net).cuda())
    y = module(x.cuda())
    with torch.no_grad():
        ref = net(x)
    assert_close(y, ref, what="MLP module")
    status_ok()


def test_mbconv_module_matches_pytorch():
    torch.manual_seed(0)
    net = MBConv()
    for p in net.parameters():
        nn.init.normal_(p, 0.0, 0.05)
    x = torch.randn(8, 24, 56, 56)
    module = DaceModule(copy.deepcopy(net).cuda())
    y = module(x.cuda())
    assert module.compiled_function.kernel_names() == ["conv2d", "conv2d", "se_gate", "conv2d"]
    with torch.no_grad():
        ref = net(x)
    assert_close(y, ref, what="MBConv module", atol=2e-5)
    status_ok()


def test_mbconv_module_half_precision():
    """The same block in fp16 (no specialised fp16 convolution kernels: the direct kernel, with the squeeze-excite
    pool taken by the row reduction in the tensors' own type); compared with PyTorch fp32 on the rounded parameters."""
    torch.manual_seed(0)
    net = MBConv()
    for p in net.parameters():
        nn.init.normal_(p, 0.0, 0.05)
    x = torch.randn(4, 24, 28, 28)
    module = DaceModule(copy.deepcopy(net).half().cuda())
    y = module(x.half().cuda())
    assert y.dtype == torch.float16
    assert module.compiled_function.kernel_names() == ["conv2d", "conv2d", "se_gate", "conv2d"]
    ref_net = copy.deepcopy(net).half().float()
    with torch.no_grad():
        ref = ref_net(x.half().float())
    assert_close(y, ref, torch.float16, what="MBConv module fp16", atol=1e-2)
    status_ok()


def test_strided_conv_module_and_decorator():
    torch.manual_seed(0)
    conv = nn.Conv2d(3, 16, 3, stride=2, bias=False)
    x = torch.randn(32, 3, 64, 64)
    y = DaceModule(copy.deepcopy(conv).cuda())(x.cuda())
    with torch.no_grad():
        assert_close(y, conv(x), what="strided conv module")

    @dace_module
    class LogSqrt(nn.Module):
        def forward(self, x):
            return torch.sqrt(torch.log(x))

    out = LogSqrt()(torch.ones(2, device="cuda"))
    assert out.tolist() == [0.0, 0.0]
    status_ok()


def test_onnx_model_multiple_outputs_keywords_and_saved_transients():
    class Two(nn.Module):
        def forward(self, x, y):
            s = x + y
            return torch.relu(s).reshape(x.shape[0], -1), torch.exp(s)

    a, b = torch.randn(4, 3, 5), torch.randn(4, 3, 5)
    saved = {}
    model = ONNXModel.from_torch("two", Two(), (a, b), save_transients=saved)
    assert model.outputs == ["__return_0", "__return_1"] and len(model.inputs) == 2
    r0, r1 = model(a.cuda(), **{model.inputs[1]: b.cuda()})
    assert_close(r0, torch.relu(a + b).reshape(4, -1), what="output 0")
    assert_close(r1, torch.exp(a + b), what="output 1")
    assert len(saved) >= 1 and all(t.is_cuda for t in saved.values())
    # host tensors are staged through the device
    h0, h1 = model(a, b)
    assert_close(h0, r0, what="host inputs")
    status_ok()


def test_lenet_module():
    """tests/torch/test_lenet.py: batch 8 of 1x32x32 images."""
    torch.manual_seed(0)
    net = LeNet()
    x = torch.rand(8, 1, 32, 32)
    module = DaceModule(copy.deepcopy(net).cuda())
    y = module(x.cuda())
    names = module.compiled_function.kernel_names()
    assert names == ["conv2d", "maxpool2d", "conv2d", "maxpool2d", "gemm", "gemm", "gemm", "softmax"]  # view(): no launch
    with torch.no_grad():
        assert_close(y, net(x), what="LeNet")
    status_ok()


def test_multihead_attention_module():
    """tests/torch/test_attn.py: ``nn.MultiheadAttention(1024, 16, bias=False)`` on [512, 2, 1024] query / key / value,
    both outputs (the attention output and the head-averaged weights)."""
    torch.manual_seed(0)
    mha = torch.nn.MultiheadAttention(1024, 16, bias=False).eval()
    q, k, v = torch.randn(512, 2, 1024), torch.randn(512, 2, 1024), torch.randn(512, 2, 1024)
    module = DaceModule(copy.deepcopy(mha).cuda())
    out, weights = module(q.cuda(), k.cuda(), v.cuda())
    with torch.no_grad():
        ref_out, ref_weights = mha(q, k, v)
    assert_close(out, ref_out, what="attention output", atol=1e-4)
    assert_close(weights, ref_weights, what="averaged attention weights", atol=1e-5)
    assert "unary" not in module.compiled_function.kernel_names()  # every reshape became a view
    status_ok()


def test_reshape_and_multiple_output_modules():
    """tests/torch/test_reshape.py and test_multi_output.py (``auto_optimize=False`` there as well)."""
    class Reshape(nn.Module):
        def forward(self, x):
            return x.reshape([5, 5])

    class TwoOutputs(nn.Module):
        def forward(self, x):
            return x + 1, x + 2

    x = torch.rand(25)
    y = DaceModule(Reshape(), auto_optimize=False, dummy_inputs=(x, ))(x.cuda())
    assert torch.equal(y.cpu(), x.reshape(5, 5))
    y = DaceModule(Reshape())(x.cuda())  # with the view pass the only node left is the copy into the output
    assert torch.equal(y.cpu(), x.reshape(5, 5))
    a, b = DaceModule(TwoOutputs(), auto_optimize=False)(x.cuda())
    assert_close(a, x + 1, what="output_0")
    assert_close(b, x + 2, what="output_1")
    status_ok()


def test_bert_encoder_reference_test_fp32():
    """tests/torch/test_bert_encoder.py:11-33: the default ``BertConfig`` layer (768 / 12 / 3072) in fp32 on
    [8, 512, 768], compared with the reference's own tolerance (rtol 1e-5, atol 1e-4).  fp32 has no fused attention
    kernel, so the graph keeps MatMul / Softmax / MatMul and the fp32 GEMM kernels."""
    layer = bert_layer(768, 12, 3072)
    torch.manual_seed(3)
    x = torch.randn(8, 512, 768)
    module = DaceModule(copy.deepcopy(layer).cuda(), training=False, simplify=True)
    y = module(x.cuda())
    names = module.compiled_function.kernel_names()
    assert "attention" not in names and names.count("softmax") == 1 and "unary" not in names
    with torch.no_grad():
        ref = layer.double()(x.double())
    ref = ref[0] if isinstance(ref, tuple) else ref
    assert_close(y, ref.float(), what="fp32 BertLayer", rtol=1e-5, atol=1e-4)
    status_ok()


def test_module_runs_through_its_torch_operator_and_under_torch_compile():
    torch.manual_seed(0)
    net = MLP()
    x = torch.randn(256, 784)
    module = DaceModule(copy.deepcopy(net).cuda(), sdfg_name="mlp_gpu_op")
    y = module(x.cuda())
    direct = torch.ops.daceml_mlp_gpu_op.mlp_gpu_op(module.torch_op_handle, x.cuda())
    assert torch.equal(y, direct)
    with torch.no_grad():
        assert_close(y, net(x), what="through the operator")

    op, handle = module.torch_op, module.torch_op_handle

    def around_op(t):
        return op(handle, t * 2.0) + 1.0

    def around_module(t):
        return module(t * 2.0) + 1.0

    with torch.no_grad():
        ref = net(x * 2.0) + 1.0
        # the operator is one opaque call inside a full graph; the module wrapper may be traced with graph breaks
        assert_close(torch.compile(around_op, backend="eager", fullgraph=True)(x.cuda()), ref, what="operator under torch.compile")
        assert_close(torch.compile(around_module, backend="eager")(x.cuda()), ref, what="module under torch.compile")
    status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_batchnorm_inference_modules(dtype):
    """BatchNorm in eval mode (running statistics): free-standing in 2-D, 3-D and 4-D, and after a convolution from a
    graph exported without the exporter's own Conv+BN folding.  Checked against the oracle and PyTorch."""
    import numpy as np
    from oracle import ops
    from daceml_b200.onnx.exported_graph import export_module
    torch.manual_seed(0)
    for bn, shape in ((nn.BatchNorm2d(24), (8, 24, 28, 28)), (nn.BatchNorm1d(40), (64, 40)), (nn.BatchNorm1d(16), (4, 16, 50))):
        bn.running_mean.normal_(), bn.running_var.uniform_(0.5, 2.0), bn.weight.data.normal_(), bn.bias.data.normal_()
        bn = bn.eval().to(dtype)
        x = torch.randn(*shape).to(dtype)
        y = DaceModule(copy.deepcopy(bn).cuda())(x.cuda())
        ref = ops.batchnorm_inference(x.float().numpy(), *(t.detach().float().numpy() for t in (bn.weight, bn.bias, bn.running_mean, bn.running_var)),
                                      eps=bn.eps)
        assert_close(y, ref, dtype=dtype, what="BatchNorm %s" % (shape, ))
        with torch.no_grad():
            assert_close(y, bn.float()(x.float()), dtype=dtype, what="BatchNorm vs torch")

    class ConvBn(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv, self.bn = nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8)

        def forward(self, x):
            return torch.relu(self.bn(self.conv(x)))

    net = ConvBn().eval()
    net.bn.running_mean.normal_(), net.bn.running_var.uniform_(0.5, 2.0)
    net = net.to(dtype)
    x = torch.randn(4, 3, 16, 16).to(dtype)
    model = ONNXModel("convbn", export_module(net, (x, ), do_constant_folding=False))
    y = model(x.cuda())
    assert model.compile_and_init().kernel_names() == ["conv2d"]
    with torch.no_grad():
        assert_close(y, net.float()(x.float()), dtype=dtype, what="Conv + BatchNorm + Relu")
    status_ok()


@pytest.mark.parametrize("stride", [1, 2])
def test_resnet_basic_block_module(stride):
    """A ResNet basic block in eval mode through ``DaceModule``: Conv 3x3 + BatchNorm + ReLU, Conv 3x3 + BatchNorm, the
    shortcut (identity, or a strided 1x1 Conv + BatchNorm) added, ReLU.  The 3x3 convolutions (and the strided 1x1) take
    the implicit-GEMM tensor-core kernel; against PyTorch in full fp32."""
    class BasicBlock(nn.Module):
        def __init__(self, cin, cout, stride):
            super().__init__()
            self.conv1, self.bn1 = nn.Conv2d(cin, cout, 3, stride=stride, padding=1, bias=False), nn.BatchNorm2d(cout)
            self.conv2, self.bn2 = nn.Conv2d(cout, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout)
            self.down = None
            if stride != 1 or cin != cout:
                self.down = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

        def forward(self, x):
            y = torch.relu(self.bn1(self.conv1(x)))
            y = self.bn2(self.conv2(y))
            return torch.relu(y + (x if self.down is None else self.down(x)))

    torch.manual_seed(0)
    net = BasicBlock(64, 64 if stride == 1 else 128, stride).eval()
    for m in net.modules():
        if isinstance(m, nn.BatchNorm2d):
            m.running_mean.normal_(0.0, 0.1), m.running_var.uniform_(0.5, 1.5), m.weight.data.uniform_(0.5, 1.5), m.bias.data.normal_(0.0, 0.1)
    x = torch.randn(8, 64, 56, 56)
    module = DaceModule(copy.deepcopy(net).cuda())
    module(x.cuda())  # builds the graph (and splits the constant weights, one small launch per convolution)
    before = L.launch_count()
    y = module(x.cuda())
    torch.cuda.synchronize()
    names = module.compiled_function.kernel_names()
    assert names.count("conv2d") == (2 if stride == 1 else 3), names
    # the weights are constants of the module: they were split for the tensor-core kernel when the module was built, so
    # every node of the graph is exactly one launch
    assert L.launch_count() - before == len(names), (L.launch_count() - before, names)
    was = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        with torch.no_grad():
            ref = net(x)
    finally:
        torch.backends.cudnn.allow_tf32 = was
    assert_close(y, ref, what="ResNet basic block, stride %d" % stride, rtol=2e-4, atol=2e-4)
    status_ok()
