#!/usr/bin/env python
"""Benchmark of the hot path: BERT-large fp16 encoder-layer samples/s on N B200s.

A step is one post-LN BERT-large encoder layer (hidden 1024, 16 heads x 64, FFN 4096, GELU erf form,
fp16 storage, fp32 accumulation) over this rank's 8 samples of 512 tokens.  Steps are chained (the
output of one is the input of the next) and cycle through 24 distinct weight sets (604 MB, larger
than L2), so K = 24 is exactly the 24-layer encoder of the multi-GPU configuration.  Ranks hold
replicated weights and exchange nothing per layer; for N > 1 the outputs are all-gathered once at the
end of the timed region.  Prints one JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH, SEQ, HIDDEN, HEADS, FFN, LAYERS = 8, 512, 1024, 16, 4096, 24
T = BATCH * SEQ
GEMM_FLOPS = {"qkv": 2 * T * HIDDEN * 3 * HIDDEN, "out": 2 * T * HIDDEN * HIDDEN, "ffn1": 2 * T * HIDDEN * FFN,
              "ffn2": 2 * T * FFN * HIDDEN}
ATTN_FLOPS = 2 * 2 * BATCH * HEADS * SEQ * SEQ * (HIDDEN // HEADS)
LAYER_FLOPS = sum(GEMM_FLOPS.values()) + ATTN_FLOPS  # 111.669 GFLOP per 8 samples
WORKLOAD = "bert-large encoder layer fp16, B=8/GPU, S=512, hidden 1024, 16 heads, FFN 4096, post-LN, GELU(erf)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


def layer_params(seed):
    g = torch.Generator().manual_seed(seed)

    def w(*s):
        return torch.randn(*s, generator=g) * 0.02
    z = torch.zeros
    return dict(wq=w(HIDDEN, HIDDEN), bq=z(HIDDEN), wk=w(HIDDEN, HIDDEN), bk=z(HIDDEN), wv=w(HIDDEN, HIDDEN), bv=z(HIDDEN),
                wo=w(HIDDEN, HIDDEN), bo=z(HIDDEN), ln1_g=torch.ones(HIDDEN), ln1_b=z(HIDDEN), w1=w(FFN, HIDDEN), b1=z(FFN),
                w2=w(HIDDEN, FFN), b2=z(HIDDEN), ln2_g=torch.ones(HIDDEN), ln2_b=z(HIDDEN))


class ClockSampler:
    """Samples SM clock, power and the clock event reasons of one GPU through NVML every few milliseconds
    while the timed region runs (reads state, changes nothing).  ``window()`` brackets the timed region;
    only samples taken inside it are reported."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, device_index):
        self.idx, self.rows, self.stop_flag, self.thread, self.h, self.nvml = device_index, [], False, None, None, None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:  # no NVML: report that instead of a clock
            self.nvml = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip() != ""]
            if self.idx < len(ids) and ids[self.idx].strip().isdigit():
                return int(ids[self.idx])
        return self.idx

    def _loop(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                self.rows.append((time.perf_counter(), n.nvmlDeviceGetClockInfo(self.h, n.NVML_CLOCK_SM),
                                  n.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(n, "nvmlDeviceGetCurrentClocksEventReasons")
                                  else n.nvmlDeviceGetCurrentClocksThrottleReasons(self.h),
                                  n.nvmlDeviceGetPowerUsage(self.h) / 1000.0))
            except Exception:
                pass
            time.sleep(0.002)

    def begin(self):
        self.t_begin = time.perf_counter()

    def end(self):
        self.t_end = time.perf_counter()

    def stop(self):
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.stop_flag = True
        self.thread.join(1.0)
        try:
            mx = float(self.nvml.nvmlDeviceGetMaxClockInfo(self.h, self.nvml.NVML_CLOCK_SM))
        except Exception:
            mx = None
        inside = [r for r in self.rows if self.t_begin is not None and self.t_begin <= r[0] <= self.t_end]
        used = inside if inside else self.rows
        reasons = set()
        for r in used:
            for bit, name in self.REASONS.items():
                if r[2] & bit:
                    reasons.add(name)
        sm = [float(r[1]) for r in used]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "in_timed_region": bool(inside),
                "power_w": float(np.median([r[3] for r in used])) if used else None}


def run_reference(args, rank):
    """The reference arm: the exported layer executed node by node on the host cores (the CPU port of the
    reference's pure expansions; its DaCe code generator is not installable here).  All 8 samples of the step, every
    core of the process's affinity mask (a launcher's OMP_NUM_THREADS=1 is overridden), rank 0 only."""
    if rank != 0:
        return
    from oracle import cpu_baseline
    params = layer_params(0)
    layer = cpu_baseline.CpuBertLayer(params, HEADS)
    x = torch.randn(BATCH, SEQ, HIDDEN, generator=torch.Generator().manual_seed(1))
    warmup = max(1, min(args.warmup, 3))
    for _ in range(warmup):
        layer.forward(x)
    steps = max(1, min(args.steps, 40))
    t0 = time.perf_counter()
    for _ in range(steps):
        layer.forward(x)
    dt = time.perf_counter() - t0
    value = BATCH * steps / dt
    out = {"impl": "reference", "metric": "bert_large_fp16_encoder_layer_samples_per_s", "value": value, "unit": "samples/s",
           "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": WORKLOAD, "sample": "all 8 samples of a step, fp32 on the host; rank 0 only, the other ranks idle",
                      "steps_asked": args.steps, "warmup_asked": args.warmup},
           "cpu_baseline": {"value": value, "unit": "samples/s", "cores": layer.threads, "kind": "port",
                            "sample": "%d steps of the layer on 8 samples (S=512), host BLAS + OpenMP loop nests" % steps},
           "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def run_hbm_kernels(args, emit=True):
    """The memory-bound kernels of the unfused BERT-large layer, each on operand sets that cycle through more than
    the 126 MB L2, timed with CUDA events over one CUDA graph: algorithmic bytes (every operand once) / time."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product path has no CPU fallback")
    from daceml_b200 import kernels as K, lib as L
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pk = peaks()
    T = BATCH * SEQ
    g = torch.Generator().manual_seed(3)

    def rnd(*shape):
        return torch.randn(*shape, generator=g).half().to(dev)

    gamma, beta, bias_h, bias_f = rnd(HIDDEN), rnd(HIDDEN), rnd(HIDDEN), rnd(FFN)
    cases = []
    n = 4  # 4 x 134 MB of scores
    sc = [rnd(BATCH * HEADS * SEQ, SEQ) for _ in range(n)]
    so = [torch.empty_like(t) for t in sc]
    cases.append(("softmax_warp_kernel", "scores [8*16*512, 512] fp16, scale 1/8", n, 2 * sc[0].numel() * 2,
                  lambda i: K.softmax(sc[i], so[i], rows=sc[i].shape[0], cols=SEQ, scale=0.125)))
    n = 24  # 24 x 25 MB
    xs, rs, ys = [rnd(T, HIDDEN) for _ in range(n)], [rnd(T, HIDDEN) for _ in range(n)], [torch.empty(T, HIDDEN, dtype=torch.float16, device=dev) for _ in range(n)]
    cases.append(("layernorm_warp_kernel", "LayerNorm(x + bias + residual) [4096, 1024] fp16", n, 3 * T * HIDDEN * 2,
                  lambda i: K.layernorm(xs[i], ys[i], gamma=gamma, beta=beta, residual=rs[i], bias=bias_h, eps=1e-12)))
    cases.append(("binary_fast_kernel", "residual add [4096, 1024] fp16", n, 3 * T * HIDDEN * 2,
                  lambda i: K.binary(xs[i], rs[i], ys[i], L.BIN_ADD)))
    # the floor at this size: a plain copy that moves the same 25 MB (12.6 MB in, 12.6 MB out) through the same launch path
    cx, cy = [rnd(T * 3 // 2, HIDDEN) for _ in range(n)], [torch.empty(T * 3 // 2, HIDDEN, dtype=torch.float16, device=dev) for _ in range(n)]
    cases.append(("unary_kernel", "plain copy of [6144, 1024] fp16: what a 25 MB launch can reach", n, 2 * (T * 3 // 2) * HIDDEN * 2,
                  lambda i: K.unary(cx[i], cy[i], L.UN_COPY)))
    n = 6  # 6 x 67 MB
    hs, ho = [rnd(T, FFN) for _ in range(n)], [torch.empty(T, FFN, dtype=torch.float16, device=dev) for _ in range(n)]
    cases.append(("bias_act_kernel", "bias + GELU(erf) [4096, 4096] fp16", n, 2 * T * FFN * 2,
                  lambda i: K.bias_act(hs[i], ho[i], bias=bias_f, act=L.EPI_GELU)))
    # the same three kernels on 8 x the rows (a batch of 64 sequences): launches long enough for the launch ramp not to count
    n, big = 3, 8 * T
    xb, rb, yb = ([rnd(big, HIDDEN) for _ in range(n)], [rnd(big, HIDDEN) for _ in range(n)],
                  [torch.empty(big, HIDDEN, dtype=torch.float16, device=dev) for _ in range(n)])
    cases.append(("layernorm_warp_kernel", "LayerNorm(x + bias + residual) [32768, 1024] fp16", n, 3 * big * HIDDEN * 2,
                  lambda i: K.layernorm(xb[i], yb[i], gamma=gamma, beta=beta, residual=rb[i], bias=bias_h, eps=1e-12)))
    cases.append(("binary_fast_kernel", "residual add [32768, 1024] fp16", n, 3 * big * HIDDEN * 2,
                  lambda i: K.binary(xb[i], rb[i], yb[i], L.BIN_ADD)))
    hb, hob = [rnd(big // 2, FFN) for _ in range(n)], [torch.empty(big // 2, FFN, dtype=torch.float16, device=dev) for _ in range(n)]
    cases.append(("bias_act_kernel", "bias + GELU(erf) [16384, 4096] fp16", n, 2 * (big // 2) * FFN * 2,
                  lambda i: K.bias_act(hb[i], hob[i], bias=bias_f, act=L.EPI_GELU)))
    # data movement: the packed QKV tensor split into its three parts (Slice on the last axis), the head-merge of two
    # halves (Concat), an embedding lookup (Gather of 1024-wide rows) and a mask select (Where)
    n = 6  # 6 x 50 MB
    qkv = [rnd(T, 3 * HIDDEN) for _ in range(n)]
    parts = [torch.empty(T, HIDDEN, dtype=torch.float16, device=dev) for _ in range(3)]

    def split3(i):
        K.strided_copy_parts([qkv[i].narrow(1, j * HIDDEN, HIDDEN) for j in range(3)], parts)

    cases.append(("strided_copy_parts_kernel", "Split of [4096, 3072] fp16 into three [4096, 1024] (1 launch)", n, 2 * T * 3 * HIDDEN * 2, split3))
    cat = [torch.empty(T, FFN, dtype=torch.float16, device=dev) for _ in range(n)]
    halves = [rnd(T, FFN // 2) for _ in range(2 * n)]

    def concat2(i):
        K.strided_copy_parts([halves[2 * i], halves[2 * i + 1]], [cat[i].narrow(1, 0, FFN // 2), cat[i].narrow(1, FFN // 2, FFN // 2)])

    cases.append(("strided_copy_parts_kernel", "Concat of two [4096, 2048] fp16 along the last axis (1 launch)", n, 2 * T * FFN * 2, concat2))
    table = rnd(30522, HIDDEN)
    ids = [torch.randint(0, 30522, (64, SEQ), generator=g).to(dev) for _ in range(4)]
    emb = [torch.empty(64, SEQ, HIDDEN, dtype=torch.float16, device=dev) for _ in range(4)]
    cases.append(("gather_kernel", "embedding lookup: [30522, 1024] fp16 table, [64, 512] ids", 4, 2 * 64 * SEQ * HIDDEN * 2 + 64 * SEQ * 8,
                  lambda i: K.gather(table, ids[i], emb[i], 0)))
    cond = [(torch.rand(T, FFN, generator=g) > 0.5).to(dev) for _ in range(n)]
    zero = torch.zeros((), dtype=torch.float16, device=dev)
    cases.append(("where_kernel", "Where(mask, x, 0) [4096, 4096] fp16, bool mask", n, T * FFN * (2 + 2 + 1),
                  lambda i: K.where(cond[i], hs[i], zero, ho[i])))
    reps = max(args.steps // 4, 12)
    rows = []
    for name, what, nset, nbytes, fn in cases:
        for i in range(min(nset, max(args.warmup, 3))):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for r in range(reps):
                fn(r % nset)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        gbs = nbytes / us / 1e3
        row = {"kernel": name, "workload": what, "launches": reps, "us_per_launch": us, "bytes_per_launch": nbytes,
               "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                            "peak_kind": "STREAM-style copy, of %s" % pk["source"]},
               "l2": "%d operand sets cycled (%.0f MB)" % (nset, nset * nbytes / 1e6)}
        rows.append(row)
        if emit:
            print(json.dumps(row), flush=True)
        del graph
    return rows


def run_other_configs(args, emit=True):
    """Configurations 1, 2 and 4 (fp32, parity cases of the test-suite) timed the same way as the layer: the compiled
    graph replayed from one CUDA graph, CUDA events around it.  `bytes` = every kernel's operands and results once."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product path has no CPU fallback")
    from daceml_b200 import graphs
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    pk = peaks()
    torch.manual_seed(0)
    rng = np.random.default_rng(4)

    def w(*shape):
        return torch.from_numpy((rng.standard_normal(shape) * 0.05).astype(np.float32))

    net = torch.nn.Sequential(torch.nn.Linear(784, 120), torch.nn.ReLU(), torch.nn.Linear(120, 32), torch.nn.ReLU(),
                              torch.nn.Linear(32, 10), torch.nn.LogSoftmax(dim=-1))
    mlp_p = {k: v.detach() for k, v in dict(w1=net[0].weight, b1=net[0].bias, w2=net[2].weight, b2=net[2].bias,
                                            w3=net[4].weight, b3=net[4].bias).items()}
    mb_p = dict(w_exp=w(144, 24, 1, 1), b_exp=w(144), w_dw=w(144, 1, 3, 3), b_dw=w(144), w_se1=w(6, 144, 1, 1), b_se1=w(6),
                w_se2=w(144, 6, 1, 1), b_se2=w(144), w_proj=w(24, 144, 1, 1), b_proj=w(24))
    cases = [
        ("config 1: Conv fp32 X[32,3,64,64] W[16,3,3,3] stride 2", graphs.conv_sdfg((32, 3, 64, 64), (16, 3, 3, 3), strides=(2, 2)).compile(),
         {"X": torch.randn(32, 3, 64, 64, device=dev), "W": torch.rand(16, 3, 3, 3, device=dev)}, "Y", (32, 16, 31, 31),
         2 * 32 * 16 * 31 * 31 * 27),
        ("config 2: MLP fp32 784-120-32-10 + LogSoftmax, batch 4096", graphs.mlp_sdfg(mlp_p, 4096, fused=True).compile(),
         {"input": torch.randn(4096, 784, device=dev)}, "__return", (4096, 10), 2 * 4096 * (784 * 120 + 120 * 32 + 32 * 10)),
        ("config 4: MBConv block fp32 [128,24,56,56], expand 144, SE 6", graphs.mbconv_sdfg(mb_p, (128, 24, 56, 56), fused=True).compile(),
         {"input": torch.randn(128, 24, 56, 56, device=dev)}, "__return", (128, 24, 56, 56),
         2 * 128 * 56 * 56 * (24 * 144 + 9 * 144 + 144 * 24)),
        # not one of the reference's configurations: a 3x3 convolution with enough channels for the implicit-GEMM kernel
        ("extra: Conv fp32 X[32,64,56,56] W[64,64,3,3] pad 1", graphs.conv_sdfg((32, 64, 56, 56), (64, 64, 3, 3), pads=(1, 1, 1, 1)).compile(),
         {"X": torch.randn(32, 64, 56, 56, device=dev), "W": torch.randn(64, 64, 3, 3, device=dev) * 0.05}, "Y", (32, 64, 56, 56),
         2 * 32 * 64 * 56 * 56 * 64 * 9),
    ]
    reps = max(args.steps // 8, 10)
    rows = []
    for name, comp, inputs, out_name, out_shape, flops in cases:
        comp.device = dev
        kw = dict(inputs)
        kw[out_name] = torch.empty(out_shape, dtype=torch.float32, device=dev)
        for _ in range(max(args.warmup, 3)):
            comp(**kw)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                comp(**kw)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps
        arrays = dict(comp._transients)
        arrays.update(comp.sdfg.constants)
        arrays.update(kw)
        nbytes, per_kernel = 0, []
        for tasklet, ins, outs in comp.plan:
            kb = 0
            for arr in list(ins.values()) + list(outs.values()):
                t = arrays.get(arr)
                if t is not None:
                    kb += t.numel() * t.element_size()
            nbytes += kb
            # the kernel on its own, same operands, one CUDA graph of `reps` launches
            call = lambda: tasklet.fn({c: arrays[n] for c, n in ins.items()}, {c: arrays[n] for c, n in outs.items()})
            g1 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                for _ in range(reps):
                    call()
            g1.replay()
            torch.cuda.synchronize()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            g1.replay()
            a1.record()
            torch.cuda.synchronize()
            kus = a0.elapsed_time(a1) * 1e3 / reps
            per_kernel.append({"kernel": "+".join(tasklet.kernels), "us": round(kus, 2), "MB": round(kb / 1e6, 2),
                               "GB/s": round(kb / kus / 1e3, 1)})
        info = None
        if name.startswith("config 1") or name.startswith("config 4") or name.startswith("extra: Conv"):
            # information only: the same arithmetic through torch's library kernels (cuDNN), the reference's GPU route
            # for convolutions (daceml/onnx/op_implementations/cudnn_implementations.py:360-379); not part of any claim
            import torch.nn.functional as Fn
            if name.startswith("config 1"):
                lib_call = lambda: Fn.conv2d(inputs["X"], inputs["W"], stride=2)
            elif name.startswith("extra: Conv"):
                lib_call = lambda: Fn.conv2d(inputs["X"], inputs["W"], padding=1)
            else:
                P = {k: v.to(dev) for k, v in mb_p.items()}
                sw = lambda t: t * torch.sigmoid(t)

                def lib_call():
                    h = sw(Fn.conv2d(inputs["input"], P["w_exp"], P["b_exp"]))
                    h = sw(Fn.conv2d(h, P["w_dw"], P["b_dw"], padding=1, groups=144))
                    g_ = torch.sigmoid(Fn.conv2d(sw(Fn.conv2d(h.mean((2, 3), keepdim=True), P["w_se1"], P["b_se1"])), P["w_se2"], P["b_se2"]))
                    return Fn.conv2d(h * g_, P["w_proj"], P["b_proj"]) + inputs["input"]
            with torch.no_grad():
                for _ in range(3):
                    lib_call()
                torch.cuda.synchronize()
                l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                l0.record()
                for _ in range(reps):
                    lib_call()
                l1.record()
                torch.cuda.synchronize()
            info = {"torch_library_kernels_us": round(l0.elapsed_time(l1) * 1e3 / reps, 2),
                    "note": "cuDNN / ATen via torch eager, information only; torch.backends.cudnn.allow_tf32 = %s (single TF32 "
                            "products, relative error 5e-4, when True)" % torch.backends.cudnn.allow_tf32}
            if name.startswith("extra: Conv"):  # the same with full fp32 products, which is what the 3 x TF32 kernel delivers
                was = torch.backends.cudnn.allow_tf32
                torch.backends.cudnn.allow_tf32 = False
                with torch.no_grad():
                    for _ in range(3):
                        lib_call()
                    torch.cuda.synchronize()
                    l0.record()
                    for _ in range(reps):
                        lib_call()
                    l1.record()
                    torch.cuda.synchronize()
                torch.backends.cudnn.allow_tf32 = was
                info["torch_library_kernels_fp32_us"] = round(l0.elapsed_time(l1) * 1e3 / reps, 2)
        row = {"workload": name, "info": info, "kernels": comp.kernel_names(), "launches_per_run": len(comp.kernel_names()),
               "per_kernel": per_kernel, "us_per_run": us, "samples_per_s": out_shape[0] / (us * 1e-6), "flops": flops, "tflops": flops / us / 1e6,
               "bytes": nbytes, "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / pk["hbm_gbs"],
               "dtype": "f32", "data": "synthetic"}
        rows.append(row)
        if emit:
            print(json.dumps(row), flush=True)
    return rows


def run_via_module(args):
    """The same metric with the layers coming from real modules: 24 HuggingFace ``BertLayer`` objects (BERT-large
    sizes, their own initialisation: normal(0, 0.02) weights, zero biases) wrapped in one ``DaceModule``.  A step is one
    layer; the 24-layer module is called ``steps / 24`` times, each call feeding the next, all in one CUDA graph timed
    with CUDA events.  Prints one JSON line (N = 1 only; no roofline probe, the kernels are those of the main run)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product path has no CPU fallback")
    import warnings
    from daceml_b200 import lib as L
    from daceml_b200.runner import upload_graph
    from daceml_b200.torch import DaceModule
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from transformers import BertConfig
        from transformers.models.bert.modeling_bert import BertLayer
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    torch.manual_seed(11)
    cfg = BertConfig(hidden_size=HIDDEN, num_attention_heads=HEADS, intermediate_size=FFN)
    cfg._attn_implementation = "eager"

    class Stack(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList([BertLayer(cfg) for _ in range(LAYERS)])

        def forward(self, x):
            for layer in self.layers:
                out = layer(x)
                x = out[0] if isinstance(out, tuple) else out
            return x

    t0 = time.perf_counter()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        module = DaceModule(Stack().half().to(dev).eval(), compile_torch_extension=False)
        x = torch.randn(BATCH, SEQ, HIDDEN, generator=torch.Generator().manual_seed(7)).half().to(dev)
        module(x)
    build_s = time.perf_counter() - t0
    compiled = module.compiled_function
    names = compiled.kernel_names()
    arg = module.sdfg.arg_names[0]
    bufs = [x.clone(), torch.empty_like(x)]
    calls = max(1, (args.steps + LAYERS - 1) // LAYERS)
    steps = calls * LAYERS

    def run(n):
        for i in range(n):
            compiled(**{arg: bufs[i % 2], "__return": bufs[(i + 1) % 2]})

    run(max(2, (args.warmup + LAYERS - 1) // LAYERS))
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run(calls)
    upload_graph(graph)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    assert L.get_context(dev).device_status() == 0 and torch.isfinite(bufs[calls % 2]).all()
    print(json.dumps({"metric": "bert_large_fp16_encoder_layer_samples_per_s", "value": BATCH * steps / (ms * 1e-3), "unit": "samples/s",
                      "n_gpus": 1, "steps": steps, "warmup": args.warmup, "ms_per_step": ms / steps, "higher_is_better": True,
                      "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "bert-large encoder layer fp16, B=8, S=512, through DaceModule(24 x transformers BertLayer)",
                                 "api": "daceml_b200.torch.DaceModule", "launches_per_layer": len(names) / LAYERS,
                                 "kernels": sorted(set(names)), "export_import_optimize_s": round(build_s, 2),
                                 "l2": "24 distinct layer weight sets (604 MB): weights come from HBM every step"},
                      "gpu_launches": len(names) * calls}), flush=True)


def replay_timed(graph, replays, after=None):
    """Replays ``graph`` ``replays`` times back to back on the current stream with a CUDA event between replays.
    ``after()`` runs after each replay (work that could not be captured).  Returns the per-replay times in ms."""
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    ev[0].record()
    for r in range(replays):
        graph.replay()
        if after is not None:
            after()
        ev[r + 1].record()
    torch.cuda.synchronize()
    return [ev[r].elapsed_time(ev[r + 1]) for r in range(replays)]


def gemm_traffic():
    """DRAM bytes per GEMM launch from the committed ncu capture (profiles/bert_large_layer_gemm_traffic.json names the
    commit and the command it was taken with); None if the file is missing."""
    path = os.path.join(ROOT, "profiles", "bert_large_layer_gemm_traffic.json")
    if not os.path.exists(path):
        return None, None
    rec = json.load(open(path))
    return rec.get("traffic_bytes_per_launch"), rec


def run_profile_kernels(args):
    """For a profiler: every kernel family of the library launched twice on operands larger than the 126 MB L2 (the
    small fp32 products excepted), nothing timed.  Used as
        ncu --section SpeedOfLight --section MemoryWorkloadAnalysis --clock-control none -c 120 python bench.py --profile-kernels
    (the second launch of each kernel is the one to read)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product path has no CPU fallback")
    from daceml_b200 import kernels as K, lib as L
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(5)
    h = lambda *s: torch.randn(*s, generator=g).half().to(dev)
    f = lambda *s: torch.randn(*s, generator=g).to(dev)
    e16 = lambda *s: torch.empty(*s, dtype=torch.float16, device=dev)
    e32 = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
    T8 = 8 * BATCH * SEQ  # 32768 rows
    jobs = []
    sc, so = h(BATCH * HEADS * SEQ, SEQ), e16(BATCH * HEADS * SEQ, SEQ)
    jobs.append(("softmax", lambda: K.softmax(sc, so, rows=sc.shape[0], cols=SEQ, scale=0.125)))
    x, r, y = h(T8, HIDDEN), h(T8, HIDDEN), e16(T8, HIDDEN)
    gam, bet, bh, bf = h(HIDDEN), h(HIDDEN), h(HIDDEN), h(FFN)
    jobs.append(("layernorm", lambda: K.layernorm(x, y, gamma=gam, beta=bet, residual=r, bias=bh, eps=1e-12)))
    jobs.append(("binary add", lambda: K.binary(x, r, y, L.BIN_ADD)))
    hx, hy = h(T8 // 2, FFN), e16(T8 // 2, FFN)
    jobs.append(("bias + gelu", lambda: K.bias_act(hx, hy, bias=bf, act=L.EPI_GELU)))
    ux, uy = f(32 << 20), e32(32 << 20)
    jobs.append(("unary sigmoid f32", lambda: K.unary(ux, uy, L.UN_SIGMOID)))
    qkv, part = h(T8, 3 * HIDDEN), e16(T8, HIDDEN)
    jobs.append(("strided copy (split)", lambda: K.strided_copy(qkv.narrow(1, HIDDEN, HIDDEN), part)))
    table, ids, emb = h(30522, HIDDEN), torch.randint(0, 30522, (128, SEQ), generator=g).to(dev), e16(128, SEQ, HIDDEN)
    jobs.append(("gather", lambda: K.gather(table, ids, emb, 0)))
    cond, zero = (torch.rand(T8 // 2, FFN, generator=g) > 0.5).to(dev), torch.zeros((), dtype=torch.float16, device=dev)
    jobs.append(("where", lambda: K.where(cond, hx, zero, hy)))
    rx, ry = f(65536, 1024), e32(65536)
    jobs.append(("reduce rows", lambda: K.reduce(rx, ry, op=L.RED_MEAN, outer=65536, red=1024, inner=1)))
    tx, ty = h(64, SEQ, HEADS, 64), e16(64, HEADS, SEQ, 64)
    jobs.append(("transpose heads", lambda: K.transpose(tx, ty, (0, 2, 1, 3))))
    cx, cy = h(64 << 20), e32(64 << 20)
    jobs.append(("cast f16 -> f32", lambda: K.cast(cx, cy)))
    ga, gw, gy = f(4096, 1024), f(1024, 1024), e32(4096, 1024)
    jobs.append(("gemm fp32 3xTF32", lambda: K.gemm(ga, gw, gy, b_layout=1)))
    sa, sw, sy = f(262144, 120), f(32, 120), e32(262144, 32)
    jobs.append(("gemm fp32 FMA", lambda: K.gemm(sa, sw, sy, b_layout=1)))
    ka, kw, ky = f(262144, 32), f(10, 32), e32(262144, 10)
    jobs.append(("gemm fp32 skinny", lambda: K.gemm(ka, kw, ky, b_layout=1)))
    c1x, c1w, c1y = f(512, 3, 64, 64), torch.rand(16, 3, 3, 3, generator=g).to(dev), e32(512, 16, 31, 31)
    jobs.append(("conv direct 3x3 stride 2", lambda: K.conv2d(c1x, c1w, c1y, strides=(2, 2))))
    mx, big, pool = f(128, 24, 56, 56), e32(128, 144, 56, 56), e32(128, 144, 1, 1)
    w_exp, b_exp = f(144, 24, 1, 1) * 0.05, f(144) * 0.05
    jobs.append(("conv 1x1 expand (tensor core)", lambda: K.conv2d(mx, w_exp, big, bias=b_exp, act=L.EPI_SWISH)))
    big2, w_dw, b_dw = e32(128, 144, 56, 56), f(144, 1, 3, 3) * 0.05, f(144) * 0.05
    jobs.append(("depthwise 3x3", lambda: K.conv2d(big, w_dw, big2, bias=b_dw, pads=(1, 1, 1, 1), group=144, act=L.EPI_SWISH, pool_mean=pool)))
    gate, w_proj, b_proj, my = torch.rand(128, 144, 1, 1, generator=g).to(dev), f(24, 144, 1, 1) * 0.05, f(24) * 0.05, e32(128, 24, 56, 56)
    jobs.append(("conv 1x1 project (tensor core)", lambda: K.conv2d(big2, w_proj, my, bias=b_proj, gate=gate, residual=mx)))
    kx, kwt, kb, ky_ = f(128, 64, 56, 56), f(64, 64, 3, 3) * 0.05, f(64) * 0.05, e32(128, 64, 56, 56)  # 103 MB in, 103 MB out
    jobs.append(("conv 3x3 implicit GEMM (tensor core)", lambda: K.conv2d(kx, kwt, ky_, bias=kb, pads=(1, 1, 1, 1), act=L.EPI_RELU)))
    for name, fn in jobs:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        print("ran", name, flush=True)
    assert L.get_context(dev).device_status() == 0


def run_gather_only(args):
    """Under torchrun: the final all-gather alone (8.4 MB per rank, the layer's output), this library's peer-store kernel
    and NCCL's collective, each as a CUDA graph of 20 launches timed with CUDA events, max over ranks.  Rank 0 prints one
    JSON line."""
    import torch.distributed as dist
    from daceml_b200 import distributed as D
    rank, world, local_rank = D.init_from_env()
    if world < 2:
        raise SystemExit("--gather-only needs torchrun with two or more ranks")
    dev = torch.device("cuda", local_rank)
    y = torch.randn(BATCH, SEQ, HIDDEN, device=dev).half()
    ref = torch.empty(world * BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev)
    peer = D.PeerGather((BATCH, SEQ, HIDDEN), torch.float16, dev, rank, world)

    def timeit(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for _ in range(n):
                    fn()
            g.replay()
            side.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            side.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del g
        return float(t)

    t_peer = timeit(lambda: peer.gather(y))
    t_nccl = timeit(lambda: dist.all_gather_into_tensor(ref, y))
    same = bool(torch.equal(peer.gathered, ref))
    if rank == 0:
        out_bytes = y.numel() * 2 * (world - 1)
        print(json.dumps({"workload": "all-gather of [8,512,1024] fp16 per rank", "n_gpus": world, "bytes_out_per_gpu": out_bytes,
                          "peer_store_kernel_us": round(t_peer, 2), "peer_store_gbs_out_per_gpu": round(out_bytes / t_peer / 1e3, 1),
                          "nccl_all_gather_us": round(t_nccl, 2), "same_result": same}), flush=True)
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    peer.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=240)
    ap.add_argument("--warmup", type=int, default=24)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="leave the fp32 configurations and the HBM-bound kernels out of the JSON line")
    ap.add_argument("--replays", type=int, default=0,
                    help="how often the K-step graph is replayed inside the timed region (default: enough for 0.15 s, at least 50)")
    ap.add_argument("--hbm-kernels", action="store_true",
                    help="instead of the layer: time the HBM-bound kernels of the unfused graph (softmax, LayerNorm, bias+GELU, "
                         "residual add) at the layer's shapes and print one JSON line per kernel with its bandwidth")
    ap.add_argument("--other-configs", action="store_true",
                    help="instead of the layer: time the fp32 configurations 1 (strided conv), 2 (MLP) and 4 (MBConv block) "
                         "at their full sizes and print one JSON line each")
    ap.add_argument("--profile-kernels", action="store_true",
                    help="instead of the layer: launch every kernel family twice on operands larger than L2, nothing timed "
                         "(the workload the ncu summaries under profiles/ were taken on)")
    ap.add_argument("--gather-only", action="store_true",
                    help="under torchrun: time the final all-gather alone, this library's peer-store kernel against NCCL")
    ap.add_argument("--via-module", action="store_true",
                    help="instead of the hand-built layer graphs: 24 transformers BertLayer modules wrapped in one DaceModule "
                         "(export, import, fusion), timed the same way; one JSON line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.gather_only:
        return run_gather_only(args)
    if args.profile_kernels:
        run_profile_kernels(args)
        return
    if args.via_module:
        run_via_module(args)
        return
    if args.hbm_kernels:
        run_hbm_kernels(args)
        return
    if args.other_configs:
        run_other_configs(args)
        return

    from daceml_b200 import distributed as D
    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the product path has no CPU fallback (use --impl reference for the CPU arm)")
    rank, world, local_rank = D.init_from_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_cores = D.bind_to_gpu_numa_node(local_rank) if world > 1 else 0
    import torch.distributed as dist
    from daceml_b200 import graphs, lib as L
    from daceml_b200.runner import upload_graph

    # ---- build: 24 fused layer SDFGs with their own weights, two ping-pong activation buffers ----
    params = [layer_params(100 + i) for i in range(LAYERS)]
    layers = []
    for i, p in enumerate(params):
        c = graphs.bert_layer_sdfg(p, BATCH, SEQ, HEADS, fused=True, name="layer%d" % i).compile()
        c.device = dev
        layers.append(c)
    kernels_per_step = len(layers[0].kernel_names())
    bufs = [torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev) for _ in range(2)]
    x0 = torch.randn(BATCH, SEQ, HIDDEN, generator=torch.Generator().manual_seed(7 + rank)).half()
    bufs[0].copy_(x0)
    gathered = torch.empty(world * BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev) if world > 1 else None
    final_buf = bufs[(args.warmup + args.steps) % 2]
    # the final all-gather: this library's kernel that stores the rank's block into every peer's memory (CUDA IPC, NVLink),
    # unless B200ML_GATHER=nccl or the mapping cannot be set up on some rank - then NCCL's collective
    peer = None
    if world > 1:
        ok = 0
        if os.environ.get("B200ML_GATHER", "peer") != "nccl":
            try:
                peer = D.PeerGather((BATCH, SEQ, HIDDEN), torch.float16, dev, rank, world)
                ok = 1
            except Exception as e:
                sys.stderr.write("rank %d: peer all-gather not available (%s)\n" % (rank, str(e).splitlines()[0] if str(e) else type(e).__name__))
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if not int(flag):
            peer = None
        if peer is not None:
            gathered = peer.gathered

    def do_gather():
        if peer is not None:
            peer.gather(final_buf)
        else:
            D.gather_outputs(final_buf, out=gathered)

    def run_steps(first, count):
        for s in range(first, first + count):
            layers[s % LAYERS](**{"input": bufs[s % 2], "__return": bufs[(s + 1) % 2]})

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def capture(first, count, gather=False):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run_steps(first, min(count, 2 * LAYERS))  # allocates transients, loads kernels
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        # thread_local: NCCL's watchdog thread polls events while this thread captures
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            run_steps(first, count)
            if gather:
                do_gather()
        return g

    if world > 1:
        do_gather()  # NCCL: creates the communicator before any capture
        barrier()
        if peer is not None:
            # the peer kernel's first result against NCCL's, on every rank, before it is trusted with the timed region
            ref = torch.empty_like(gathered)
            dist.all_gather_into_tensor(ref, final_buf)
            torch.cuda.synchronize()
            good = int(torch.equal(ref, peer.gathered) and L.get_context(dev).device_status() == 0)
            flag = torch.tensor([good], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if not int(flag):
                sys.stderr.write("rank %d: peer all-gather disagreed with NCCL or left a status; using NCCL\n" % rank)
                peer, gathered = None, ref
            barrier()
    warm_graph = capture(0, args.warmup)
    gather_in_graph = False
    if world > 1:
        # the one all-gather of the outputs rides in the same CUDA graph as the K steps, so no host launch sits between
        # the last layer and the collective; every rank must agree on whether that worked
        try:
            timed_graph = capture(args.warmup, args.steps, gather=True)
            ok = 1
        except Exception as e:  # capture of the collective refused: issue it from the host behind each replay
            sys.stderr.write("rank %d: all-gather not captured (%s)\n" % (rank, str(e).splitlines()[0] if str(e) else type(e).__name__))
            torch.cuda.synchronize()
            ok = 0
        flag = torch.tensor([ok], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        gather_in_graph = bool(int(flag))
        if not gather_in_graph:
            timed_graph = capture(args.warmup, args.steps)
    else:
        timed_graph = capture(args.warmup, args.steps)
    uploaded = upload_graph(timed_graph)  # the first replay is a timed one: the upload must not be part of it
    after = None
    if world > 1 and not gather_in_graph:
        after = do_gather

    # ---- device-timed region: W warm-up steps, then the K-step graph R times back to back ----
    barrier()
    bufs[0].copy_(x0)
    warm_graph.replay()
    est = replay_timed(timed_graph, 2, after)[-1]
    replays = args.replays
    if replays <= 0:
        replays = int(min(400, max(50, np.ceil(150.0 / max(est, 1e-3)))))
    if world > 1:
        rt = torch.tensor([replays], device=dev)
        dist.all_reduce(rt, op=dist.ReduceOp.MAX)
        replays = int(rt)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    bufs[0].copy_(x0)
    warm_graph.replay()  # the W untimed steps, straight before the timed ones
    barrier()
    sampler.begin()
    t_host = time.perf_counter()
    times = replay_timed(timed_graph, replays, after)
    host_ms = (time.perf_counter() - t_host) * 1e3
    barrier()
    sampler.end()
    if world > 1:
        tt = torch.tensor(times, device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)  # a replay takes as long as its slowest rank
        times = tt.tolist()
    clocks = sampler.stop() if rank == 0 else None
    status = L.get_context(dev).device_status()
    assert torch.isfinite(final_buf).all(), "non-finite activations"
    med = float(np.median(times))
    ms_per_step = med / args.steps
    value = world * BATCH * args.steps / (med * 1e-3)

    # ---- contents of the gathered output: own block bit for bit, every other block against its owner's checksum ----
    gather_checked = None
    if world > 1:
        mine = gathered[rank * BATCH:(rank + 1) * BATCH]
        same = bool(torch.equal(mine, final_buf))
        sums = gathered.view(torch.int16).to(torch.int64).view(world, -1)
        weights = torch.arange(1, sums.shape[1] + 1, device=dev, dtype=torch.int64) % 65521
        seen = (sums * weights).sum(dim=1)  # position-weighted, so a permutation inside a block shows as well
        own = (final_buf.view(torch.int16).to(torch.int64).view(-1) * weights).sum().view(1)
        owners = torch.empty(world, dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(owners, own)
        ok = torch.tensor([int(same and bool(torch.equal(seen, owners)))], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        gather_checked = bool(int(ok))
        assert gather_checked, "the gathered output does not hold every rank's block in rank order"
        # what the collective alone costs (its own graph-free launch, events around it), for the record
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(10):
            do_gather()
        g1.record()
        torch.cuda.synchronize()
        gather_ms = g0.elapsed_time(g1) / 10

    # ---- roofline of the dominant kernel (the tcgen05 GEMM) ----
    # Events cannot sit between the kernels of the timed graph without opening gaps in it, so each GEMM of the step is
    # timed in a CUDA graph of its own: the same launch, once for each of the 24 layers (that layer's weights and
    # buffers), replayed 20 times with events around each replay; the median replay counts.  Launches follow one another as
    # they do in the step (programmatic dependent launch included); what is lost is the L2 residency of the activations
    # the previous kernel of the step wrote.
    pk = peaks()
    gemm_us, per_gemm = 0.0, []
    plan0 = layers[0].plan
    for ti, (tasklet0, _, _) in enumerate(plan0):
        if not tasklet0.kernels[0].startswith("gemm"):
            continue

        def run_tasklet():
            for s in range(LAYERS):
                comp = layers[s]
                tasklet, ins, outs = comp.plan[ti]
                arrays = dict(comp._transients)
                arrays.update(comp.sdfg.constants)
                arrays.update({"input": bufs[s % 2], "__return": bufs[(s + 1) % 2]})
                tasklet.fn({c: arrays[n] for c, n in ins.items()}, {c: arrays[n] for c, n in outs.items()})

        run_tasklet()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run_tasklet()
        g.replay()
        torch.cuda.synchronize()
        us = float(np.median(replay_timed(g, 20))) * 1e3 / LAYERS
        per_gemm.append({"tasklet": tasklet0.label, "kernel": tasklet0.kernels[0], "us": us})
        gemm_us += us
    n_gemm = len(per_gemm)
    gemm_flops = sum(GEMM_FLOPS.values())
    achieved_tf = gemm_flops / (gemm_us * 1e-6) / 1e12 if gemm_us > 0 else None
    step_tf = LAYER_FLOPS / (ms_per_step * 1e-3) / 1e12
    # which measured peak applies: the burst figure when the SM clock held (within 5 %) at its maximum through the timed
    # region, the sustained (power-capped) figure otherwise; both fractions are printed either way
    held = bool(clocks and clocks.get("in_timed_region") and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                and clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"]) if rank == 0 else False
    peak_kind, peak_tf = ("burst", pk["tf_burst"]) if held else ("sustained", pk["tf_sustained"])
    traffic, traffic_rec = gemm_traffic()
    roofline = {"bound": "tensor", "kernel": "tcgen05 GEMM kernels (gemm_f16_pair_kernel x2, gemm_f16_ln_kernel x2 per layer)",
                "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved_tf / peak_tf if achieved_tf else None,
                "frac_burst": achieved_tf / pk["tf_burst"] if achieved_tf else None,
                "frac_sustained": achieved_tf / pk["tf_sustained"] if achieved_tf else None,
                "peak_kind": "%s cuBLAS bf16, of %s (SM clock in the timed region: %s of %s MHz)" % (
                    peak_kind, pk["source"], clocks.get("sm_mhz") if clocks else None, clocks.get("sm_max_mhz") if clocks else None),
                "launches_timed": n_gemm * LAYERS * 20,
                "avg_launch_us": gemm_us / max(n_gemm, 1), "flops_per_launch": gemm_flops / max(n_gemm, 1),
                "per_launch_us": {p["tasklet"]: round(p["us"], 2) for p in per_gemm},
                "probe": "each GEMM of the step in a CUDA graph of its own, 24 launches (one per layer), median of 20 replays, CUDA events",
                "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum, mean of the 4 GEMM launches of a layer)",
                "traffic_source": traffic_rec,
                "whole_step": {"tflops": step_tf, "frac": step_tf / peak_tf, "frac_burst": step_tf / pk["tf_burst"],
                               "frac_sustained": step_tf / pk["tf_sustained"], "flops_per_step": LAYER_FLOPS}}

    # ---- end to end through the public API with host buffers: H2D of the step's input, layer, D2H of its output ----
    n_e2e = 240  # long enough (about 50 ms) for the fill and drain of the three-deep pipeline (about 0.5 ms) not to count
    depth = 3
    hin = [torch.randn(BATCH, SEQ, HIDDEN).half().pin_memory() for _ in range(depth)]
    hout = [torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16).pin_memory() for _ in range(depth)]
    din = [torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev) for _ in range(depth)]
    dout = [torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev) for _ in range(depth)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def pipeline(step_graphs):
        """H2D, compute and D2H on three streams over ``depth`` buffer sets; step i uses set i % depth."""
        def run(n):
            ev_in, ev_cmp, ev_out = [None] * depth, [None] * depth, [None] * depth
            for i in range(n):
                j = i % depth
                with torch.cuda.stream(s_in):
                    if ev_cmp[j] is not None:
                        s_in.wait_event(ev_cmp[j])  # the step that read din[j] has finished
                    din[j].copy_(hin[j], non_blocking=True)
                    ev_in[j] = torch.cuda.Event()
                    ev_in[j].record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(ev_in[j])
                    if ev_out[j] is not None:
                        s_cmp.wait_event(ev_out[j])  # dout[j] has been copied out
                    step_graphs[j].replay()
                    ev_cmp[j] = torch.cuda.Event()
                    ev_cmp[j].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[j])
                    hout[j].copy_(dout[j], non_blocking=True)
                    ev_out[j] = torch.cuda.Event()
                    ev_out[j].record(s_out)
        return run

    def timed_passes(run, n):
        """Three wall-clock passes of ``run(n)`` (max over ranks each); the median."""
        run(depth * 2)
        torch.cuda.synchronize()
        out = []
        for _ in range(3):
            barrier()
            t0 = time.perf_counter()
            run(n)
            torch.cuda.synchronize()
            t = time.perf_counter() - t0
            if world > 1:
                te = torch.tensor([t], device=dev)
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
                t = float(te)
            out.append(t)
        return sorted(out)[1], out

    layer_graphs = []
    for j in range(depth):
        with torch.cuda.stream(s_cmp):
            layers[j % LAYERS](**{"input": din[j], "__return": dout[j]})
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s_cmp):
            layers[j % LAYERS](**{"input": din[j], "__return": dout[j]})
        layer_graphs.append(g)
    # on these hosts the pipeline settles into one of two states from pass to pass (PCIe copies in both directions
    # under the layer's HBM traffic), hence three passes and their median
    e2e_s, e2e_runs = timed_passes(pipeline(layer_graphs), n_e2e)
    nbytes = BATCH * SEQ * HIDDEN * 2
    e2e = {"value": world * BATCH * n_e2e / e2e_s, "unit": "samples/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
           "steps": n_e2e, "pipeline": "3 buffers; copy-in, layer and copy-out on separate streams",
           "passes_samples_per_s": [round(world * BATCH * n_e2e / t) for t in e2e_runs], "reported": "median of 3 passes"}

    # ---- the same end to end at the granularity of the 24-layer encoder: one copy in, 24 layers, one copy out ----
    stack_graphs = []
    for j in range(depth):
        tmp = torch.empty(BATCH, SEQ, HIDDEN, dtype=torch.float16, device=dev)

        def stack(j=j, tmp=tmp):
            src = din[j]
            for s in range(LAYERS):
                dst = dout[j] if s == LAYERS - 1 else (tmp if s % 2 == 0 else din[j])
                layers[s](**{"input": src, "__return": dst})
                src = dst

        # 24 layers: even count, so the chain din -> tmp -> din ... ends in tmp before the last layer writes dout
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s_cmp):
            stack()
        stack_graphs.append(g)
    n_passes = 12
    c5_s, c5_runs = timed_passes(pipeline(stack_graphs), n_passes)
    e2e_config5 = {"value": world * BATCH * LAYERS * n_passes / c5_s, "unit": "samples/s (layer-steps, as the headline)",
                   "encoder_samples_per_s": world * BATCH * n_passes / c5_s, "h2d_bytes_per_pass": nbytes, "d2h_bytes_per_pass": nbytes,
                   "passes": n_passes, "layers_per_pass": LAYERS,
                   "what": "one pinned H2D of [8,512,1024] fp16, the 24-layer encoder, one D2H, pipelined over 3 buffer sets",
                   "passes_samples_per_s": [round(world * BATCH * LAYERS * n_passes / t) for t in c5_runs]}

    # ---- CPU baseline beside it (rank 0, N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import cpu_baseline
        sps, iters, threads = cpu_baseline.time_layer(params[0], HEADS, batch=BATCH, seq=SEQ, budget_s=12.0)
        cpu = {"value": sps, "unit": "samples/s", "cores": threads, "kind": "port",
               "sample": "%d runs of the layer on all 8 samples (S=512), fp32, host BLAS + OpenMP loop nests" % iters}

    # ---- the other configurations and the HBM-bound kernels, so that one line records them (N = 1 only) ----
    other_configs = hbm_kernels = None
    if rank == 0 and world == 1 and not args.no_extras:
        timed_graph = warm_graph = layer_graphs = stack_graphs = None
        torch.cuda.empty_cache()
        sub = argparse.Namespace(steps=96, warmup=3)
        other_configs = [{"workload": r["workload"], "us_per_run": round(r["us_per_run"], 2), "bytes": r["bytes"],
                          "gbs": round(r["gbs"], 1), "frac_of_hbm_peak": round(r["frac_of_hbm_peak"], 4),
                          "tflops": round(r["tflops"], 3), "launches_per_run": r["launches_per_run"], "per_kernel": r["per_kernel"],
                          "info": r.get("info")}
                         for r in run_other_configs(sub, emit=False)]
        hbm_kernels = [{"kernel": r["kernel"], "workload": r["workload"], "us_per_launch": round(r["us_per_launch"], 2),
                        "bytes_per_launch": r["bytes_per_launch"], "gbs": round(r["roofline"]["achieved"], 1),
                        "frac_of_hbm_peak": round(r["roofline"]["frac"], 4)} for r in run_hbm_kernels(sub, emit=False)]

    if rank == 0:
        if clocks is not None and clocks.get("sm_mhz"):
            clocks["ms_per_step_x_sm_mhz"] = ms_per_step * clocks["sm_mhz"]
        out = {"metric": "bert_large_fp16_encoder_layer_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "f16", "data": "synthetic",
               "config": {"workload": WORKLOAD, "global_batch": world * BATCH, "seq_len": SEQ, "parallelism": "dp%d" % world,
                          "l2": "24 distinct layer weight sets (604 MB) cycled: weights come from HBM every step",
                          "chained": True,
                          "graph": "the K timed steps are one CUDA graph" + (", uploaded to the device (cudaGraphUpload) before the timed region" if uploaded else ""),
                          "timed_region": "the K-step graph replayed %d times back to back, a CUDA event between replays; ms_per_step = median replay / K" % replays,
                          "gather": ("one all-gather of the final outputs per replay, " + ("captured in the same CUDA graph as the K steps" if gather_in_graph else "issued from the host behind the replay")) if world > 1 else "none",
                          "numa": ("process bound to the %d cores next to its GPU" % numa_cores) if numa_cores else "not bound"},
               "replays": replays, "steps_timed_total": replays * args.steps,
               "replay_ms": {"median": med, "min": float(np.min(times)), "max": float(np.max(times)), "mean": float(np.mean(times)),
                             "p10": float(np.percentile(times, 10)), "p90": float(np.percentile(times, 90))},
               "timed_region_ms": float(np.sum(times)), "timed_region_host_ms": host_ms,
               "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_config5": e2e_config5,
               "gpu_launches": kernels_per_step * args.steps * replays + (replays if peer is not None else 0),
               "kernels_per_step": kernels_per_step, "clocks": clocks, "device_status": status,
               "peaks": pk}
        if world > 1:
            out["gather_checked"] = gather_checked
            out["gather_ms"] = gather_ms
            out["gather_method"] = ("b200ml_peer_allgather: one kernel per rank, 16-byte stores into the peers' memory (CUDA IPC) over NVLink"
                                    if peer is not None else "NCCL all_gather_into_tensor")
            out["gather_bytes_per_rank"] = nbytes
        if other_configs is not None:
            out["other_configs"] = other_configs
            out["hbm_kernels"] = hbm_kernels
        print(json.dumps(out), flush=True)
    if world > 1:
        # A communicator cannot be torn down while CUDA graphs that hold its collectives are alive: drop them first.
        # Should the teardown still stall, the line is printed already and nothing is in flight: leave after 30 s.
        guard = threading.Timer(30.0, lambda: os._exit(0))
        guard.daemon = True
        guard.start()
        timed_graph = warm_graph = layer_graphs = stack_graphs = None
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        if peer is not None:
            peer.close()
        dist.destroy_process_group()
        guard.cancel()


if __name__ == "__main__":
    main()
