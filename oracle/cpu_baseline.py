"""Timed CPU baseline: the exported BERT encoder layer executed node by node on the host cores.

TEST / BASELINE INFRASTRUCTURE ONLY (used by ``bench.py`` and the tests; never by the product).

This is what the reference's CPU path does after ``auto_optimize``: every MatMul goes to the BLAS
library node (``daceml/util/utils.py:226-229``; torch's CPU BLAS stands in for OpenBLAS here), and
every other ONNX node is its own OpenMP loop nest with the tensor written to memory in between
(the loop nests are in ``cpu_ops.c``).  The reference's own DaCe-generated code cannot be produced
here (DaCe is not installed), so ``kind`` is ``"port"``.
"""
import ctypes
import math
import os
import subprocess
import time

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "liboracle_cpu.so")


def build():
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
    return _LIB


def load():
    if not os.path.exists(_LIB):
        build()
    lib = ctypes.CDLL(_LIB)
    f32p, i64 = ctypes.POINTER(ctypes.c_float), ctypes.c_int64
    lib.conv2d_nchw.argtypes = [f32p, f32p, f32p, f32p] + [i64] * 14
    lib.softmax_rows.argtypes = [f32p, f32p, i64, i64, ctypes.c_int]
    lib.reduce_mean_rows.argtypes = [f32p, f32p, i64, i64]
    lib.ew_binary.argtypes = [f32p, f32p, f32p, i64, i64, ctypes.c_int, ctypes.c_int]
    lib.ew_unary.argtypes = [f32p, f32p, i64, ctypes.c_int]
    lib.transpose4d.argtypes = [f32p, f32p, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    lib.oracle_num_threads.restype = ctypes.c_int
    lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
    return lib


def host_cores():
    """The cores this process may run on (its affinity mask), whatever OMP_NUM_THREADS says."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _p(t):
    return ctypes.cast(t.data_ptr(), ctypes.POINTER(ctypes.c_float))


class CpuBertLayer:
    """fp32 tensors, node-by-node; ``forward(x)`` with x [B, S, H] float32 (torch, CPU)."""

    def __init__(self, params, heads, eps=1e-12):
        self.lib = load()
        self.p = {k: v.detach().float().contiguous() for k, v in params.items() if v is not None}
        self.heads, self.eps = heads, eps
        # every core of the affinity mask, for the loop nests (OpenMP) and for the BLAS calls (torch): a launcher's
        # OMP_NUM_THREADS=1 must not shrink the baseline to one core
        self.lib.oracle_set_num_threads(host_cores())
        self.threads = int(self.lib.oracle_num_threads())
        torch.set_num_threads(max(self.threads, 1))

    # one ONNX node each
    def _binary(self, a, b, op, mode):
        y = torch.empty_like(a)
        rows = a.numel() // a.shape[-1]
        self.lib.ew_binary(_p(a), _p(b), _p(y), rows, a.shape[-1], op, mode)
        return y

    def _unary(self, x, op):
        y = torch.empty_like(x)
        self.lib.ew_unary(_p(x), _p(y), x.numel(), op)
        return y

    def _transpose(self, x, perm):
        y = torch.empty([x.shape[i] for i in perm], dtype=torch.float32)
        shape = (ctypes.c_int64 * 4)(*x.shape)
        pm = (ctypes.c_int64 * 4)(*perm)
        self.lib.transpose4d(_p(x), _p(y), shape, pm)
        return y

    def _linear(self, x, w, b):
        wt = w.t().contiguous()                                  # Transpose(W, [1, 0])
        mm = torch.matmul(x, wt)                                 # MatMul -> BLAS
        return self._binary(mm, b, 0, 2)                         # Add(bias)

    def _layernorm(self, x, g, b):
        rows, cols = x.numel() // x.shape[-1], x.shape[-1]
        mean = torch.empty(rows)
        self.lib.reduce_mean_rows(_p(x), _p(mean), rows, cols)   # ReduceMean
        d = self._binary(x, mean, 1, 1)                          # Sub
        two = torch.tensor([2.0])
        sq = self._binary(d, two, 4, 3)                          # Pow
        var = torch.empty(rows)
        self.lib.reduce_mean_rows(_p(sq), _p(var), rows, cols)   # ReduceMean
        epst = torch.tensor([self.eps], dtype=torch.float32)
        ve = self._binary(var.view(1, -1), epst, 0, 3).view(-1)  # Add(eps)
        std = self._unary(ve, 1)                                 # Sqrt
        nrm = self._binary(d, std, 3, 1)                         # Div
        sc = self._binary(nrm, g, 2, 2)                          # Mul(gamma)
        return self._binary(sc, b, 0, 2)                         # Add(beta)

    def forward(self, x):
        p, h = self.p, self.heads
        B, S, H = x.shape
        d = H // h
        q = self._transpose(self._linear(x, p["wq"], p["bq"]).view(B, S, h, d), (0, 2, 1, 3))
        k = self._transpose(self._linear(x, p["wk"], p["bk"]).view(B, S, h, d), (0, 2, 3, 1))
        v = self._transpose(self._linear(x, p["wv"], p["bv"]).view(B, S, h, d), (0, 2, 1, 3))
        scores = torch.matmul(q, k)                                              # MatMul -> batched BLAS
        scores = self._binary(scores, torch.tensor([1.0 / math.sqrt(d)]), 2, 3)  # Mul(0.125)
        probs = torch.empty_like(scores)
        self.lib.softmax_rows(_p(scores), _p(probs), B * h * S, S, 0)            # Softmax
        ctx = torch.matmul(probs, v)                                             # MatMul
        ctx = self._transpose(ctx, (0, 2, 1, 3)).view(B, S, H)
        attn = self._binary(self._linear(ctx, p["wo"], p["bo"]), x, 0, 0)        # Add(residual)
        h1 = self._layernorm(attn, p["ln1_g"], p["ln1_b"])
        f = self._linear(h1, p["w1"], p["b1"])
        gd = self._binary(f, torch.tensor([1.41421354]), 3, 3)                   # Div
        ge = self._unary(gd, 0)                                                  # Erf
        ga = self._binary(ge, torch.tensor([1.0]), 0, 3)                         # Add(1)
        gm = self._binary(f, ga, 2, 0)                                           # Mul(x)
        inter = self._binary(gm, torch.tensor([0.5]), 2, 3)                      # Mul(0.5)
        out = self._binary(self._linear(inter, p["w2"], p["b2"]), h1, 0, 0)
        return self._layernorm(out, p["ln2_g"], p["ln2_b"])


def conv2d(x, w, b=None, strides=(1, 1), pads=(0, 0, 0, 0), group=1):
    """The 7-deep loop nest through ctypes; numpy float32 arrays."""
    lib = load()
    n, c, h, wd = x.shape
    m, _, kh, kw = w.shape
    oh = (h + pads[0] + pads[2] - kh) // strides[0] + 1
    ow = (wd + pads[1] + pads[3] - kw) // strides[1] + 1
    y = np.empty((n, m, oh, ow), dtype=np.float32)
    f32p = ctypes.POINTER(ctypes.c_float)
    x, w = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(w, np.float32)
    bp = np.ascontiguousarray(b, np.float32).ctypes.data_as(f32p) if b is not None else None
    lib.conv2d_nchw(x.ctypes.data_as(f32p), w.ctypes.data_as(f32p), bp, y.ctypes.data_as(f32p), n, c, h, wd, m, kh, kw,
                    strides[0], strides[1], pads[0], pads[1], pads[2], pads[3], group)
    return y


def time_layer(params, heads, batch, seq, budget_s=15.0, warmup=1, min_iters=2):
    """Runs the layer on ``batch`` samples repeatedly for about ``budget_s`` seconds.

    Returns ``(samples_per_s, iterations, threads)``."""
    layer = CpuBertLayer(params, heads)
    hidden = params["wq"].shape[0]
    x = torch.randn(batch, seq, hidden, generator=torch.Generator().manual_seed(1))
    for _ in range(warmup):
        layer.forward(x)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_iters or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        layer.forward(x)
        times.append(time.perf_counter() - t0)
        if len(times) >= 200:
            break
    med = sorted(times)[len(times) // 2]
    return batch / med, len(times), layer.threads
