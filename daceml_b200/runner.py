"""Running compiled SDFGs repeatedly: static buffers, CUDA-graph replay, layer stacks.

The reference compiles an SDFG once and keeps a state handle so that later calls only pass
pointers (``daceml/torch/dispatchers/common.py:34-76``).  The counterpart here is a launch plan
captured into a CUDA graph: the Python side of each step is one ``cudaGraphLaunch``.
"""
from typing import List, Optional

import torch

from daceml_b200 import graphs
from daceml_b200 import lib as L


def upload_graph(graph: "torch.cuda.CUDAGraph") -> bool:
    """``cudaGraphUpload``: moves an instantiated graph to the device ahead of its first replay, which otherwise pays
    for the upload (about 1.6 us per kernel node).  Returns False when the CUDA Python bindings are missing."""
    try:
        from cuda.bindings import runtime as cudart
        err = cudart.cudaGraphUpload(graph.raw_cuda_graph_exec(), torch.cuda.current_stream().cuda_stream)[0]
        torch.cuda.synchronize()
        return err == cudart.cudaError_t.cudaSuccess
    except Exception:
        return False


class GraphedCall:
    """Captures ``fn()`` (kernel launches on the current stream over static buffers) in a CUDA graph."""

    def __init__(self, fn, warmup=2):
        self.fn = fn
        self.graph = None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            fn()
        self.uploaded = upload_graph(self.graph)

    def __call__(self):
        self.graph.replay()


class BertEncoder:
    """A stack of post-LN BERT encoder layers over one batch shard, fp16 storage / fp32 accumulation.

    Each layer is the fused SDFG of :func:`daceml_b200.graphs.bert_layer_sdfg` with its own weights
    bound as constants; activations ping-pong between two static buffers, so a forward pass is
    ``7 * layers`` kernel launches and no allocation."""

    def __init__(self, layer_params: List[dict], batch, seq, heads, device=None, fused=True, cuda_graph=True,
                 eps=1e-12):
        if not torch.cuda.is_available():
            raise L.B200Error(L.ERR_CUDA, "BertEncoder needs a B200; there is no CPU path")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.batch, self.seq, self.heads = batch, seq, heads
        self.hidden = layer_params[0]["wq"].shape[0]
        shape = (batch, seq, self.hidden)
        self.buffers = [torch.zeros(shape, dtype=torch.float16, device=self.device) for _ in range(2)]
        self.layers = []
        with torch.cuda.device(self.device):
            for i, p in enumerate(layer_params):
                s = graphs.bert_layer_sdfg(p, batch, seq, heads, fused=fused, eps=eps, name="bert_layer_%d" % i)
                c = s.compile()
                c.device = self.device
                self.layers.append(c)
            self.launches_per_forward = sum(len(c.kernel_names()) for c in self.layers)
            self._graphed: Optional[GraphedCall] = None
            self._cuda_graph = cuda_graph
            if cuda_graph:
                self._graphed = GraphedCall(self._run_layers)

    @property
    def input_buffer(self):
        return self.buffers[0]

    @property
    def output_buffer(self):
        return self.buffers[len(self.layers) % 2]

    def _run_layers(self):
        for i, layer in enumerate(self.layers):
            # a dict, because a "__return" keyword inside a class body would be name-mangled
            layer(**{"input": self.buffers[i % 2], "__return": self.buffers[(i + 1) % 2]})

    def forward_static(self):
        """Runs the stack on whatever is in ``input_buffer``; the result is in ``output_buffer``."""
        if self._graphed is not None:
            self._graphed()
        else:
            self._run_layers()
        return self.output_buffer

    def __call__(self, x):
        """``x``: [batch, seq, hidden] fp16 on any device; returns the output buffer (device tensor)."""
        self.input_buffer.copy_(x, non_blocking=True)
        return self.forward_static()
