"""ctypes binding of ``libdaceml_b200.so`` (declared in ``include/daceml_b200.h``).

The reference reaches native code the same way: it generates a C bridge, builds a shared library
and loads it with ctypes (``daceml/ort_api/raw_api_bindings.py:273-321``); opaque handles travel as
integers (``daceml/torch/dispatchers/common.py:76``).  There is no CPU path behind these calls: if
the library is missing or no B200 is visible, importing succeeds but the first call raises.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# DACEML_B200_LIB selects another build of the same library (e.g. an instrumented one)
LIB_PATH = os.environ.get("DACEML_B200_LIB") or os.path.join(_HERE, "lib", "libdaceml_b200.so")

# status codes / enums (mirrors of the header)
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE, ERR_WORKSPACE = 0, -1, -2, -3, -4, -5
F16, F32, I64, I32, F64, U8, BOOL = range(7)
EPI_BIAS, EPI_RELU, EPI_GELU, EPI_RESIDUAL, EPI_SWISH, EPI_LAYERNORM = 1, 2, 4, 8, 16, 32
GEMM_B_CONSTANT = 1
RED_SUM, RED_MEAN, RED_MAX, RED_MIN = 0, 1, 2, 3
(UN_COPY, UN_RELU, UN_SIGMOID, UN_ERF, UN_SQRT, UN_EXP, UN_LOG, UN_TANH, UN_SWISH, UN_GELU, UN_RECIPROCAL,
 UN_LEAKYRELU, UN_AFFINE, UN_POWS, UN_SOFTPLUS, UN_CLIP, UN_NEG, UN_ABS) = range(18)
BIN_ADD, BIN_SUB, BIN_MUL, BIN_DIV, BIN_POW, BIN_MAX, BIN_MIN = range(7)
CMP_EQ, CMP_GT, CMP_LT, CMP_GE, CMP_LE = range(5)

EXPORTED_SYMBOLS = [
    "b200ml_ctx_create", "b200ml_ctx_destroy", "b200ml_ctx_device_status", "b200ml_ctx_workspace_bytes",
    "b200ml_last_error", "b200ml_version", "b200ml_launch_count", "b200ml_gemm", "b200ml_softmax",
    "b200ml_layernorm", "b200ml_reduce", "b200ml_reduce_static", "b200ml_unary", "b200ml_binary", "b200ml_bias_act", "b200ml_transpose",
    "b200ml_cast", "b200ml_conv2d", "b200ml_se_gate", "b200ml_attention_f16", "b200ml_strided_copy", "b200ml_gather",
    "b200ml_where", "b200ml_compare", "b200ml_maxpool2d", "b200ml_wait_probe", "b200ml_strided_copy_parts",
    "b200ml_peer_allgather", "b200ml_ipc_export", "b200ml_ipc_open", "b200ml_ipc_close",
    "b200ml_conv_prepack_bytes", "b200ml_conv_prepack",
]


class B200Error(RuntimeError):
    """A libdaceml_b200 call failed; ``code`` is the negative status it returned."""

    def __init__(self, code, message):
        super().__init__(f"libdaceml_b200 error {code}: {message}")
        self.code = code


class Unsupported(B200Error):
    """The library has no kernel for this (valid) request; expansions report "cannot be applied"."""


MAX_PEERS = 16


class PeerGroup(ctypes.Structure):
    """b200ml_peer_group of include/daceml_b200.h."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32), ("gathered", ctypes.c_void_p * MAX_PEERS),
                ("flags", ctypes.c_void_p * MAX_PEERS)]


class GemmParams(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("a_layout", ctypes.c_int32), ("b_layout", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("batch_outer", ctypes.c_int64), ("batch_inner", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("a_stride_outer", ctypes.c_int64), ("a_stride_inner", ctypes.c_int64),
        ("ldb", ctypes.c_int64), ("b_stride_outer", ctypes.c_int64), ("b_stride_inner", ctypes.c_int64),
        ("ldc", ctypes.c_int64), ("c_stride_outer", ctypes.c_int64), ("c_stride_inner", ctypes.c_int64),
        ("ldr", ctypes.c_int64), ("r_stride_outer", ctypes.c_int64), ("r_stride_inner", ctypes.c_int64),
        ("alpha", ctypes.c_float), ("bias_scale", ctypes.c_float), ("residual_scale", ctypes.c_float),
        ("flags", ctypes.c_int32),
        ("a", ctypes.c_void_p), ("b", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
        ("c", ctypes.c_void_p),
        ("ln_gamma", ctypes.c_void_p), ("ln_beta", ctypes.c_void_p), ("ln_eps", ctypes.c_float), ("reserved2", ctypes.c_int32),
    ]


class ConvParams(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("act", ctypes.c_int32),
        ("n", ctypes.c_int64), ("c", ctypes.c_int64), ("h", ctypes.c_int64), ("w", ctypes.c_int64),
        ("m", ctypes.c_int64), ("kh", ctypes.c_int64), ("kw", ctypes.c_int64),
        ("stride_h", ctypes.c_int64), ("stride_w", ctypes.c_int64),
        ("pad_top", ctypes.c_int64), ("pad_left", ctypes.c_int64), ("pad_bottom", ctypes.c_int64),
        ("pad_right", ctypes.c_int64),
        ("dil_h", ctypes.c_int64), ("dil_w", ctypes.c_int64), ("group", ctypes.c_int64),
        ("x", ctypes.c_void_p), ("weight", ctypes.c_void_p), ("bias", ctypes.c_void_p), ("gate", ctypes.c_void_p),
        ("residual", ctypes.c_void_p), ("y", ctypes.c_void_p), ("pool_sum", ctypes.c_void_p),
        ("packed_weight", ctypes.c_void_p),
    ]


class AttentionParams(ctypes.Structure):
    _fields_ = [
        ("batch", ctypes.c_int64), ("heads", ctypes.c_int64), ("seq_q", ctypes.c_int64), ("seq_kv", ctypes.c_int64),
        ("head_dim", ctypes.c_int64),
        ("q_stride_b", ctypes.c_int64), ("q_stride_h", ctypes.c_int64), ("q_stride_s", ctypes.c_int64),
        ("k_stride_b", ctypes.c_int64), ("k_stride_h", ctypes.c_int64), ("k_stride_s", ctypes.c_int64),
        ("v_stride_b", ctypes.c_int64), ("v_stride_h", ctypes.c_int64), ("v_stride_s", ctypes.c_int64),
        ("o_stride_b", ctypes.c_int64), ("o_stride_h", ctypes.c_int64), ("o_stride_s", ctypes.c_int64),
        ("scale", ctypes.c_float), ("reserved", ctypes.c_int32),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("mask", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
    ]


_lib = None
_lib_lock = threading.Lock()


def load_library(path=None):
    """Loads the shared library (once) and declares every entry point's signature."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    with _lib_lock:
        if _lib is not None and path is None:
            return _lib
        p = path or LIB_PATH
        if not os.path.exists(p):
            raise ImportError(
                f"{p} is missing: build it with `python -m daceml_b200.build` (nvcc, sm_100a). "
                "daceml_b200 has no CPU or eager fallback.")
        lib = ctypes.CDLL(p)
        c_i32, c_i64, c_f, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
        i64p, i32p = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int32)
        lib.b200ml_ctx_create.argtypes = [ctypes.c_int, c_i64, ctypes.POINTER(vp)]
        lib.b200ml_ctx_destroy.argtypes = [vp]
        lib.b200ml_ctx_device_status.argtypes = [vp, i32p]
        lib.b200ml_ctx_workspace_bytes.argtypes = [vp]
        lib.b200ml_ctx_workspace_bytes.restype = c_i64
        lib.b200ml_last_error.restype = ctypes.c_char_p
        lib.b200ml_launch_count.restype = c_i64
        lib.b200ml_gemm.argtypes = [vp, ctypes.POINTER(GemmParams), vp]
        lib.b200ml_softmax.argtypes = [vp, c_i32, vp, vp, vp, c_i64, c_i64, c_i64, c_f, c_i32, vp]
        lib.b200ml_layernorm.argtypes = [vp, c_i32, vp, vp, vp, vp, vp, vp, c_i64, c_i64, c_f, vp]
        lib.b200ml_reduce.argtypes = [vp, c_i32, c_i32, vp, vp, c_i64, c_i64, c_i64, vp]
        lib.b200ml_reduce_static.argtypes = [c_i32, c_i32, vp, vp, c_i64, c_i64, c_i64, vp]
        lib.b200ml_unary.argtypes = [vp, c_i32, c_i32, vp, vp, c_i64, c_f, c_f, vp]
        lib.b200ml_binary.argtypes = [vp, c_i32, c_i32, vp, vp, vp, c_i32, i64p, i64p, i64p, vp]
        lib.b200ml_bias_act.argtypes = [vp, c_i32, vp, vp, vp, vp, c_i64, c_i64, c_i32, vp]
        lib.b200ml_transpose.argtypes = [vp, c_i32, vp, vp, c_i32, i64p, i32p, vp]
        lib.b200ml_cast.argtypes = [vp, c_i32, c_i32, vp, vp, c_i64, vp]
        lib.b200ml_conv2d.argtypes = [vp, ctypes.POINTER(ConvParams), vp]
        lib.b200ml_conv_prepack_bytes.argtypes = [vp, ctypes.POINTER(ConvParams)]
        lib.b200ml_conv_prepack_bytes.restype = ctypes.c_int64
        lib.b200ml_conv_prepack.argtypes = [vp, ctypes.POINTER(ConvParams), vp, vp]
        lib.b200ml_se_gate.argtypes = [vp, c_i32, vp, vp, vp, vp, vp, vp, c_i64, c_i64, c_i64, vp]
        lib.b200ml_attention_f16.argtypes = [vp, ctypes.POINTER(AttentionParams), vp]
        lib.b200ml_strided_copy.argtypes = [vp, c_i32, vp, vp, c_i32, i64p, i64p, i64p, vp]
        lib.b200ml_gather.argtypes = [vp, c_i32, vp, vp, vp, c_i64, c_i64, c_i64, c_i64, vp]
        lib.b200ml_where.argtypes = [vp, c_i32, vp, vp, vp, vp, c_i32, i64p, i64p, i64p, i64p, vp]
        lib.b200ml_compare.argtypes = [vp, c_i32, c_i32, vp, vp, vp, c_i32, i64p, i64p, i64p, vp]
        lib.b200ml_maxpool2d.argtypes = [vp, c_i32, vp, vp, c_i64, c_i64, c_i64] + [c_i32] * 8 + [vp]
        lib.b200ml_wait_probe.argtypes = [vp, c_i64, vp, vp]
        lib.b200ml_strided_copy_parts.argtypes = [vp, c_i32, c_i32, ctypes.POINTER(vp), ctypes.POINTER(vp), c_i32, i64p, i64p, i64p, vp]
        lib.b200ml_peer_allgather.argtypes = [vp, ctypes.POINTER(PeerGroup), vp, c_i64, vp]
        lib.b200ml_ipc_export.argtypes = [vp, vp, vp, i64p]
        lib.b200ml_ipc_open.argtypes = [vp, vp, c_i64, ctypes.POINTER(vp)]
        lib.b200ml_ipc_close.argtypes = [vp, vp, c_i64]
        for name in EXPORTED_SYMBOLS:
            fn = getattr(lib, name)
            if name not in ("b200ml_last_error", "b200ml_launch_count", "b200ml_ctx_workspace_bytes", "b200ml_conv_prepack_bytes"):
                fn.restype = ctypes.c_int
        if path is None:
            _lib = lib
        return lib


def check(code):
    """Turns a negative status into a Python exception carrying the library's message."""
    if code == OK:
        return
    msg = load_library().b200ml_last_error().decode("utf-8", "replace")
    if code == ERR_UNSUPPORTED:
        raise Unsupported(code, msg)
    raise B200Error(code, msg)


def launch_count():
    return int(load_library().b200ml_launch_count())


def dtype_code(dt):
    if dt == torch.float16:
        return F16
    if dt == torch.float32:
        return F32
    raise Unsupported(ERR_UNSUPPORTED, f"dtype {dt} has no B200 kernel (float16 and float32 only)")


CAST_CODES = {torch.float16: F16, torch.float32: F32, torch.int64: I64, torch.int32: I32, torch.float64: F64, torch.uint8: U8,
              torch.bool: BOOL}


def cast_code(dt):
    """The dtype code of an operand of ``b200ml_cast`` (a wider set than the arithmetic kernels take)."""
    if dt not in CAST_CODES:
        raise Unsupported(ERR_UNSUPPORTED, f"dtype {dt} cannot be cast on the device")
    return CAST_CODES[dt]


class Context:
    """One per (process, device): the analogue of ``CudnnHandle::Get(device)``."""

    def __init__(self, device=0, workspace_bytes=64 << 20):
        self.lib = load_library()
        self.device = int(device)
        handle = ctypes.c_void_p()
        check(self.lib.b200ml_ctx_create(self.device, int(workspace_bytes), ctypes.byref(handle)))
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self.lib.b200ml_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def device_status(self):
        """Synchronises nothing; call after the stream is idle.  Raises if a kernel gave up a wait."""
        st = ctypes.c_int32(0)
        check(self.lib.b200ml_ctx_device_status(self.handle, ctypes.byref(st)))
        return st.value


_contexts = {}
_override = threading.local()


class use_context:
    """``with use_context(ctx):`` makes the calls of this thread go through ``ctx`` instead of the process-wide context
    of its device.  A context's scratch buffer serves one call at a time on the GPU, so work that runs on several
    streams at once gives each stream a context of its own (``Context(device)``)."""

    def __init__(self, ctx):
        self.ctx = ctx

    def __enter__(self):
        self.previous = getattr(_override, "ctx", None)
        _override.ctx = self.ctx
        return self.ctx

    def __exit__(self, *exc):
        _override.ctx = self.previous


def get_context(device=None):
    """The process-wide context of a CUDA device (created on first use), or the one ``use_context`` put in its place."""
    over = getattr(_override, "ctx", None)
    if over is not None:
        index = device.index if isinstance(device, torch.device) else device
        if index is None or index == over.device:
            return over
    if device is None:
        if not torch.cuda.is_available():
            raise B200Error(ERR_CUDA, "no CUDA device is visible; daceml_b200 has no CPU path")
        device = torch.cuda.current_device()
    elif isinstance(device, torch.device):
        device = device.index if device.index is not None else torch.cuda.current_device()
    ctx = _contexts.get(device)
    if ctx is None:
        ctx = _contexts[device] = Context(device)
    return ctx


def current_stream(device=None):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None
