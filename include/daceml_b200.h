/*
 * daceml_b200.h -- C ABI of libdaceml_b200.so
 *
 * A B200 (sm_100a) implementation of the forward path of DaCeML's ONNX operator
 * library nodes.  Every entry point below is what a DaCeML expansion
 * (an ONNXForward subclass registered with @op_implementation) binds instead of
 * returning a nested SDFG: the expansion hands over raw device pointers, extents
 * and attributes, exactly as the reference's generated tasklets hand them to
 * cuDNN or ONNX Runtime.
 *
 * Conventions (borrowed from the reference where it has one):
 *   - Tensors are C-contiguous unless a stride argument says otherwise; the
 *     caller owns all memory and pre-allocates outputs
 *     (daceml/onnx/onnx_importer.py:585-590, daceml/torch/dispatchers/ctypes_module.py:58-67).
 *   - One context per (process, device), the analogue of
 *     daceml::cudnn::CudnnHandle::Get(device) (daceml/onnx/include/daceml_cudnn.h:41-62).
 *     A context is not thread-safe, and calls on ONE context must not overlap on
 *     the GPU: the fp32 tensor-core GEMM (its split operands) and the long-row
 *     reduction (its partial results) use the context's scratch buffer, so two
 *     such calls running at once on different streams would overwrite each
 *     other's scratch.  Work on several streams at once uses one context per stream.
 *   - Kernels are enqueued on the stream passed in and never synchronise the host
 *     (the reference sets state.nosync, daceml/torch/dispatchers/cpp_torch_extension.py:474-475).
 *   - Every function returns 0 on success or a negative b200ml_status; the message
 *     is available from b200ml_last_error().  Nothing prints-and-exits as
 *     __ort_check_status does (daceml/onnx/include/dace_onnx.h:7-15).
 *   - Device-side waits are bounded.  A kernel that gave up records a code in the
 *     context's status word, readable with b200ml_ctx_device_status() after the
 *     stream has been synchronised.
 */
#ifndef DACEML_B200_H
#define DACEML_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200ml_ctx b200ml_ctx;
typedef void* b200ml_stream; /* a cudaStream_t */

typedef enum {
    B200ML_OK = 0,
    B200ML_ERR_INVALID = -1,     /* bad argument (null pointer, negative extent, misaligned) */
    B200ML_ERR_UNSUPPORTED = -2, /* valid ONNX, but no kernel here: the expansion must say "cannot be applied" */
    B200ML_ERR_CUDA = -3,        /* a CUDA runtime / driver call failed */
    B200ML_ERR_DEVICE = -4,      /* a kernel recorded a device-side error (bounded wait ran out) */
    B200ML_ERR_WORKSPACE = -5    /* the context's scratch buffer is too small */
} b200ml_status;

typedef enum {
    B200ML_F16 = 0,
    B200ML_F32 = 1,
    /* the types below are accepted by b200ml_cast (all of them) and b200ml_compare (B200ML_I64) only */
    B200ML_I64 = 2,
    B200ML_I32 = 3,
    B200ML_F64 = 4,
    B200ML_U8 = 5,
    B200ML_BOOL = 6 /* one byte, 0 / 1; casting to it tests x != 0 */
} b200ml_dtype;

/* ------------------------------------------------------------------------- */
/* Context and errors                                                         */
/* ------------------------------------------------------------------------- */

/* Replaces CudnnHandle::Get(device) (daceml/onnx/include/daceml_cudnn.h:41-62) and the
 * per-SDFG init code of daceml/onnx/environments/cudnn.py:33-49.  Allocates the
 * context's scratch buffer (workspace_bytes, may be 0) and its status word. */
int b200ml_ctx_create(int device, int64_t workspace_bytes, b200ml_ctx** out);
int b200ml_ctx_destroy(b200ml_ctx* ctx);
/* Reads (and clears) the device status word.  Call after synchronising the stream. */
int b200ml_ctx_device_status(b200ml_ctx* ctx, int32_t* status);
int64_t b200ml_ctx_workspace_bytes(const b200ml_ctx* ctx);
/* Diagnostic, no counterpart in the reference (whose status helpers print and exit, dace_onnx.h:7-15): runs the
 * give-up path of the library's bounded device-side waits on purpose.  One CTA waits, for at most limit_ns
 * (1 ns .. 100 ms), on an mbarrier that nothing completes; when the limit runs out it records a code in the
 * context's status word and the kernel ends normally.  After synchronising the stream,
 * b200ml_ctx_device_status() returns B200ML_ERR_DEVICE with status 6 and clears the word; the context and the
 * device stay usable.  waited_us (device memory, may be null) receives the time the CTA spent waiting. */
int b200ml_wait_probe(b200ml_ctx* ctx, int64_t limit_ns, uint32_t* waited_us, b200ml_stream stream);
/* Replaces __ort_check_status / CheckCudnnError (dace_onnx.h:7-15, daceml_cudnn.h:17-24). */
const char* b200ml_last_error(void);
int b200ml_version(void);
/* Number of kernels this library has launched in the calling process (all contexts). */
int64_t b200ml_launch_count(void);

/* ------------------------------------------------------------------------- */
/* MatMul / Gemm / Einsum-as-matmul                                           */
/* ------------------------------------------------------------------------- */

/* Epilogue: out = act(alpha * (A.B) + bias_scale * bias[n]) + residual_scale * residual[m, n] */
enum {
    B200ML_EPI_BIAS = 1,
    B200ML_EPI_RELU = 2,
    B200ML_EPI_GELU = 4, /* 0.5 x (1 + erf(x / sqrt 2)), the Div/Erf/Add/Mul/Mul chain */
    B200ML_EPI_RESIDUAL = 8,
    B200ML_EPI_SWISH = 16, /* x * sigmoid(x), the Sigmoid/Mul pair */
    /* LayerNorm over the N axis of the finished row (after bias / activation / residual), with ln_gamma, ln_beta and
     * ln_eps: the ReduceMean/Sub/Pow/ReduceMean/Add/Sqrt/Div/Mul/Add chain folded into the GEMM.  F16 only, N a
     * multiple of 256 up to 1024; other shapes return B200ML_ERR_UNSUPPORTED (run b200ml_layernorm after the GEMM). */
    B200ML_EPI_LAYERNORM = 32
};

/* b200ml_gemm_params.flags.  B_CONSTANT: nothing enqueued earlier on the stream writes B (a weight bound when the
 * graph was built, as DaCeML binds parameters, daceml/onnx/onnx_importer.py:256-297).  The fp16 tensor-core kernels
 * then fetch the first pipeline stages of B before they wait for the preceding kernel to finish (programmatic
 * dependent launch): the weights stream in under the predecessor's tail.  Leave it 0 for a B that is an activation. */
#define B200ML_GEMM_B_CONSTANT 1

typedef struct {
    int32_t dtype;    /* B200ML_F16: tcgen05 tensor cores, fp32 accumulate, fp16 in/out.
                         B200ML_F32: FP32 FMA (no TF32 rounding). */
    int32_t a_layout; /* 0: A is [M,K] row-major. 1: A is stored [K,M] (Gemm transA=1); F32 only. */
    int32_t b_layout; /* 0: B is [K,N] row-major (ONNX MatMul). 1: B is stored [N,K] (Gemm transB=1, nn.Linear weight). */
    int32_t epilogue; /* B200ML_EPI_* flags */
    int64_t m, n, k;
    int64_t batch_outer, batch_inner; /* two batch loops (e.g. B and heads); 1 when unused */
    /* element strides: leading dimension, then per batch loop (0 broadcasts an operand) */
    int64_t lda, a_stride_outer, a_stride_inner;
    int64_t ldb, b_stride_outer, b_stride_inner;
    int64_t ldc, c_stride_outer, c_stride_inner;
    int64_t ldr, r_stride_outer, r_stride_inner;
    float alpha, bias_scale, residual_scale;
    int32_t flags; /* B200ML_GEMM_B_CONSTANT or 0 */
    const void* a;
    const void* b;
    const void* bias;     /* [N] or null */
    const void* residual; /* [M,N] with ldr, or null */
    void* c;
    const void* ln_gamma; /* [N] or null (B200ML_EPI_LAYERNORM) */
    const void* ln_beta;  /* [N] or null */
    float ln_eps;
    int32_t reserved2;
} b200ml_gemm_params;

/* Replaces PureMatMul / PureEinsum / PureGemm and the BLAS library node they lower to
 * (daceml/onnx/op_implementations/pure_implementations.py:111-252, 380-553). */
int b200ml_gemm(b200ml_ctx* ctx, const b200ml_gemm_params* p, b200ml_stream stream);

/* ------------------------------------------------------------------------- */
/* Row-wise kernels                                                           */
/* ------------------------------------------------------------------------- */

/* y[r,:] = softmax(scale * x[r,:] + mask[r / mask_row_div, :]) over contiguous rows
 * (log_softmax when is_log != 0).  mask may be null.  Replaces Softmax / LogSoftmax
 * (pure_implementations.py:309-319, 649-656) and the Mul(0.125) / Add(mask) nodes in front. */
int b200ml_softmax(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* mask, void* y,
                   int64_t rows, int64_t cols, int64_t mask_row_div, float scale, int32_t is_log,
                   b200ml_stream stream);

/* y = (v - mean(v)) / sqrt(mean((v-mean)^2) + eps) * gamma + beta with v = x (+ residual) (+ bias[cols]).
 * Replaces the ReduceMean/Sub/Pow/ReduceMean/Add/Sqrt/Div/Mul/Add chain
 * (pure_implementations.py:34-41, 76-103) and the residual Add in front of it. */
int b200ml_layernorm(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* residual,
                     const void* bias, const void* gamma, const void* beta, void* y, int64_t rows,
                     int64_t cols, float eps, b200ml_stream stream);

typedef enum { B200ML_RED_SUM = 0, B200ML_RED_MEAN = 1, B200ML_RED_MAX = 2, B200ML_RED_MIN = 3 } b200ml_reduce_op;

/* x viewed as [outer, reduce, inner]; y[outer, inner] = op over the middle extent.
 * Replaces ReduceSum/Mean/Max/Min (pure_implementations.py:101-103, 294-306) and
 * GlobalAveragePool (img_op_implementations.py:415-526). */
int b200ml_reduce(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* x, void* y, int64_t outer,
                  int64_t reduce, int64_t inner, b200ml_stream stream);

/* The same reduction for callers that may not allocate device memory: no context is needed, and the
 * scratch for the per-slice partial results of long rows is a 4 KiB array built into the library
 * (resident on every GPU that loads it, until the process exits) instead of a cudaMalloc'ed buffer.
 * Meant for code running under CUDA-graph capture or inside a serving loop (where cudaMalloc would
 * synchronise the device or is illegal), and for plug-ins whose host framework fixes their memory
 * budget.  It has no counterpart in the reference.
 *   - Works on the current device and the given stream; calls no allocating routine.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call before any stream capture begins.
 *   - Limit: outer * slices <= 1024 partial results.  Rows are sliced only when reduce > 4096 and
 *     outer < 4 * SM count, into ceil(4 * SMs / outer) slices (at most reduce / 2048); on a B200 only
 *     513..591 long rows at once exceed the limit.  Such a request fails with B200ML_ERR_WORKSPACE
 *     and a message; b200ml_reduce with a context serves it.
 *   - All calls share the one array and it keeps the last call's partials; nothing has to be
 *     zeroed, but two calls that overlap on the GPU (different streams) race on it. */
int b200ml_reduce_static(int32_t dtype, int32_t op, const void* x, void* y, int64_t outer,
                         int64_t reduce, int64_t inner, b200ml_stream stream);

/* ------------------------------------------------------------------------- */
/* Element-wise kernels                                                       */
/* ------------------------------------------------------------------------- */

typedef enum {
    B200ML_UN_COPY = 0,
    B200ML_UN_RELU = 1,
    B200ML_UN_SIGMOID = 2,
    B200ML_UN_ERF = 3,
    B200ML_UN_SQRT = 4,
    B200ML_UN_EXP = 5,
    B200ML_UN_LOG = 6,
    B200ML_UN_TANH = 7,
    B200ML_UN_SWISH = 8,      /* x * sigmoid(x) */
    B200ML_UN_GELU = 9,       /* erf form */
    B200ML_UN_RECIPROCAL = 10,
    B200ML_UN_LEAKYRELU = 11, /* max(x,0) + p0 * min(x,0) */
    B200ML_UN_AFFINE = 12,    /* p0 * x + p1 */
    B200ML_UN_POWS = 13,      /* x ** p0 */
    B200ML_UN_SOFTPLUS = 14,
    B200ML_UN_CLIP = 15,      /* min(max(x, p0), p1) */
    B200ML_UN_NEG = 16,
    B200ML_UN_ABS = 17
} b200ml_unary_op;

/* Replaces the dace.elementwise bodies of pure_implementations.py:24-36, 106-108, 283-291,
 * 556-568, 736-743. */
int b200ml_unary(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* x, void* y, int64_t n,
                 float p0, float p1, b200ml_stream stream);

typedef enum {
    B200ML_BIN_ADD = 0,
    B200ML_BIN_SUB = 1,
    B200ML_BIN_MUL = 2,
    B200ML_BIN_DIV = 3,
    B200ML_BIN_POW = 4,
    B200ML_BIN_MAX = 5,
    B200ML_BIN_MIN = 6
} b200ml_binary_op;

/* Numpy-broadcast binary op.  shape is the output shape (rank <= 6); a_strides / b_strides are
 * element strides of the operands in that shape, 0 on broadcast dimensions.  Replaces
 * Add/Sub/Mul/Div/Pow (pure_implementations.py:39-41, 76-93). */
int b200ml_binary(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* a, const void* b, void* y,
                  int32_t rank, const int64_t* shape, const int64_t* a_strides,
                  const int64_t* b_strides, b200ml_stream stream);

/* y[r,c] = act(x[r,c] + bias[c]) (+ residual[r,c]); act is a B200ML_EPI_* activation flag or 0.
 * The stand-alone form of the GEMM epilogue (bias Add followed by Relu / the GELU chain). */
int b200ml_bias_act(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* bias,
                    const void* residual, void* y, int64_t rows, int64_t cols, int32_t act,
                    b200ml_stream stream);

/* y = permute(x, perm) for elements of elem_bytes (2 or 4), rank <= 6.  Replaces Transpose and
 * EinsumTranspose (pure_implementations.py:322-326, 746-778). */
int b200ml_transpose(b200ml_ctx* ctx, int32_t elem_bytes, const void* x, void* y, int32_t rank,
                     const int64_t* shape, const int32_t* perm, b200ml_stream stream);

/* Replaces Cast (pure_implementations.py:329-377): any pair of b200ml_dtype values; float -> integer truncates toward
 * zero, anything -> B200ML_BOOL tests x != 0. */
int b200ml_cast(b200ml_ctx* ctx, int32_t src_dtype, int32_t dst_dtype, const void* x, void* y,
                int64_t n, b200ml_stream stream);

/* ------------------------------------------------------------------------- */
/* Data movement: Slice / Split / Concat / Expand, Gather, Where, MaxPool      */
/* ------------------------------------------------------------------------- */

/* y[sum_d i_d * y_strides[d]] = x[sum_d i_d * x_strides[d]] for every index i of shape (rank <= 6); strides are in
 * elements of elem_bytes (1, 2, 4 or 8), x strides may be 0 (broadcast), and x / y already point at the first element
 * (the caller adds a slice's offset).  One entry point for the copies the reference writes as memlet sub-ranges:
 * Slice (pure_implementations.py:659-735, 830-904; any axes and positive steps here, axis 0 / step 1 there),
 * Split (:781-827), Expand (:260-281; a real broadcast here, only the no-op case there) and Concat. */
int b200ml_strided_copy(b200ml_ctx* ctx, int32_t elem_bytes, const void* x, void* y, int32_t rank,
                        const int64_t* shape, const int64_t* x_strides, const int64_t* y_strides,
                        b200ml_stream stream);

/* The same for up to eight copies of one element size in a single launch: part p copies shapes[p * rank ...] from xs[p]
 * to ys[p] with its own strides.  This is Split (pure_implementations.py:781-827: one sub-range copy per output) and
 * Concat as one kernel instead of one per part; parts that cannot move the same unit fall back to one launch each. */
int b200ml_strided_copy_parts(b200ml_ctx* ctx, int32_t elem_bytes, int32_t nparts, const void* const* xs,
                              void* const* ys, int32_t rank, const int64_t* shapes, const int64_t* x_strides,
                              const int64_t* y_strides, b200ml_stream stream);

/* numpy.take along one axis: data is [outer, axis_dim, inner], y is [outer, n_indices, inner],
 * y[o, j, :] = data[o, indices[j], :]; negative indices count from the end.  An index outside [-axis_dim, axis_dim)
 * writes zeros and sets the context's device status.  Replaces Gather (pure_implementations.py:949-1014). */
int b200ml_gather(b200ml_ctx* ctx, int32_t elem_bytes, const void* data, const int64_t* indices, void* y,
                  int64_t outer, int64_t axis_dim, int64_t inner, int64_t n_indices, b200ml_stream stream);

/* out = condition ? x : y with numpy broadcasting: shape is the output shape (contiguous, rank <= 6), the strides are
 * those of the operands in that shape (0 on broadcast axes); condition holds one byte per element.  Replaces Where
 * (pure_implementations.py:96-98). */
int b200ml_where(b200ml_ctx* ctx, int32_t elem_bytes, const void* condition, const void* x, const void* y, void* out,
                 int32_t rank, const int64_t* shape, const int64_t* c_strides, const int64_t* x_strides,
                 const int64_t* y_strides, b200ml_stream stream);

typedef enum b200ml_compare_op {
    B200ML_CMP_EQ = 0,
    B200ML_CMP_GT = 1,
    B200ML_CMP_LT = 2,
    B200ML_CMP_GE = 3,
    B200ML_CMP_LE = 4
} b200ml_compare_op;

/* out = a <op> b as one byte per element (0 / 1) with numpy broadcasting (strides as in b200ml_binary); dtype is
 * B200ML_F16, B200ML_F32 or B200ML_I64.  Equal / Greater / Less (and the -OrEqual forms of opset 12), which produce the
 * condition of a Where; the reference leaves these to its ONNX Runtime fallback. */
int b200ml_compare(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* a, const void* b, void* out,
                   int32_t rank, const int64_t* shape, const int64_t* a_strides, const int64_t* b_strides,
                   b200ml_stream stream);

/* 2-D max pooling over [planes = N*C, h, w], floor mode, no dilation; padding reads as -infinity and must be smaller
 * than the kernel.  Replaces MaxPool (img_op_implementations.py:28-161, which has no padding). */
int b200ml_maxpool2d(b200ml_ctx* ctx, int32_t dtype, const void* x, void* y, int64_t planes, int64_t h, int64_t w,
                     int32_t kh, int32_t kw, int32_t stride_h, int32_t stride_w, int32_t pad_top, int32_t pad_left,
                     int32_t pad_bottom, int32_t pad_right, b200ml_stream stream);

/* ------------------------------------------------------------------------- */
/* Convolution and squeeze-excite                                             */
/* ------------------------------------------------------------------------- */

typedef struct {
    int32_t dtype; /* B200ML_F32 (B200ML_F16 storage with fp32 accumulate also accepted) */
    int32_t act;   /* 0, B200ML_EPI_RELU or B200ML_EPI_SWISH applied after bias */
    int64_t n, c, h, w;  /* X is [n, c, h, w] */
    int64_t m, kh, kw;   /* W is [m, c / group, kh, kw] */
    int64_t stride_h, stride_w;
    int64_t pad_top, pad_left, pad_bottom, pad_right;
    int64_t dil_h, dil_w;
    int64_t group;
    const void* x;
    const void* weight;   /* [m, c / group, kh, kw] */
    const void* bias;     /* [m] or null */
    const void* gate;     /* [n, c] or null: X is multiplied by gate[n, c] on load (squeeze-excite) */
    const void* residual; /* [n, m, oh, ow] or null, added after act */
    void* y;              /* [n, m, oh, ow] */
    float* pool_sum;      /* [n, m] or null: receives the mean of y over (oh, ow) (GlobalAveragePool fused) */
    const void* packed_weight; /* null, or what b200ml_conv_prepack wrote for these weights, bias and shapes */
} b200ml_conv_params;

/* ONNX Conv (cross-correlation, NCHW).  Replaces PureConv2D (img_op_implementations.py:164-330)
 * for stride 1 / no pad / group 1, and CudnnConvolution (cudnn_implementations.py:123-410) for
 * strided, padded and grouped convolutions.  fp32 group-1 convolutions run on the tensor cores at
 * fp32 accuracy (three TF32 products per term): stride-1 1x1 kernels with 8..256 output channels,
 * and kernels up to 7 x 7 with stride 1 or 2 whose reduction has 64 terms or more as an implicit GEMM; both use
 * the context's scratch for the split weights, so calls sharing a context must not overlap. */
int b200ml_conv2d(b200ml_ctx* ctx, const b200ml_conv_params* p, b200ml_stream stream);
/* Weights that do not change between calls can be prepared once (the role cuDNN's filter descriptors and a framework's
 * weight pre-packing play for the reference's GPU route, cudnn_implementations.py:205-240): the tensor-core kernels
 * want weight and bias split into their TF32 hi and lo parts and re-ordered, which b200ml_conv2d otherwise does with a
 * small kernel at every call.  b200ml_conv_prepack_bytes returns the size of the packed form for this convolution (its
 * tensor pointers are not read), 0 if the convolution runs on a kernel that takes the weights as they are.
 * b200ml_conv_prepack writes it (16-byte aligned device memory of that size, owned by the caller); later calls pass it
 * as p->packed_weight together with the same weight, bias, shapes and attributes. */
int64_t b200ml_conv_prepack_bytes(b200ml_ctx* ctx, const b200ml_conv_params* p);
int b200ml_conv_prepack(b200ml_ctx* ctx, const b200ml_conv_params* p, void* packed, b200ml_stream stream);

/* gate[n, c] = sigmoid(W2 . swish(W1 . pooled[n, :] + b1) + b2): the two 1x1 convolutions of a
 * squeeze-excite block on a [n, c, 1, 1] tensor.  w1 is [r, c], w2 is [c, r]. */
int b200ml_se_gate(b200ml_ctx* ctx, int32_t dtype, const void* pooled, const void* w1,
                   const void* b1, const void* w2, const void* b2, void* gate, int64_t n, int64_t c,
                   int64_t r, b200ml_stream stream);

/* ------------------------------------------------------------------------- */
/* Multi-GPU: all-gather of the ranks' outputs over peer memory               */
/* ------------------------------------------------------------------------- */

/* No counterpart in the reference (it has no multi-device path).  One process per GPU; the batch is split over the
 * ranks and their outputs are gathered once at the end.  Every rank allocates a gathered buffer
 * ([world][bytes_per_rank], 16-byte aligned) and 64 zero-initialised uint32 flag words, exports them with
 * b200ml_ipc_export, sends handle and offset to its peers through whatever channel the host program has, and maps the
 * peers' with b200ml_ipc_open (CUDA IPC: device memory obtained from cudaMalloc, all processes on one box). */
#define B200ML_MAX_PEERS 16
typedef struct {
    int32_t rank, world;
    void* gathered[B200ML_MAX_PEERS];    /* [r]: rank r's gathered buffer as mapped in this process ([rank] is this rank's own) */
    void* flags[B200ML_MAX_PEERS];       /* [r]: rank r's 64 flag words as mapped in this process */
} b200ml_peer_group;

/* Every rank calls this once per step, in the same order on every rank: src (bytes_per_rank bytes, a multiple of 16)
 * lands in slot [rank] of every rank's gathered buffer by plain 16-byte stores over NVLink; when the kernel has
 * completed on a rank, that rank's gathered buffer holds every rank's block.  A rank does not overwrite a peer's
 * buffer before that peer has entered the same step on its stream.  The waits on the peers' flags are bounded (1 s):
 * a peer that never arrives leaves status 7 in the context's status word (b200ml_ctx_device_status) instead of a hang.
 * The launch can be captured in a CUDA graph and replayed (the step counter lives in the flag words). */
int b200ml_peer_allgather(b200ml_ctx* ctx, const b200ml_peer_group* group, const void* src, int64_t bytes_per_rank,
                          b200ml_stream stream);
/* handle64 receives the 64-byte CUDA IPC handle of the allocation that holds ptr, *offset ptr's offset inside it. */
int b200ml_ipc_export(b200ml_ctx* ctx, const void* ptr, void* handle64, int64_t* offset);
/* Maps the allocation behind a peer's handle into this process and returns the address that corresponds to the
 * peer's ptr; enables peer access from this context's device as needed.  Not for handles of this same process. */
int b200ml_ipc_open(b200ml_ctx* ctx, const void* handle64, int64_t offset, void** ptr);
int b200ml_ipc_close(b200ml_ctx* ctx, void* ptr, int64_t offset);

/* ------------------------------------------------------------------------- */
/* Fused attention                                                            */
/* ------------------------------------------------------------------------- */

typedef struct {
    int64_t batch, heads, seq_q, seq_kv, head_dim;
    /* element strides of q, k, v, o per (batch, head, position); head_dim is contiguous */
    int64_t q_stride_b, q_stride_h, q_stride_s;
    int64_t k_stride_b, k_stride_h, k_stride_s;
    int64_t v_stride_b, v_stride_h, v_stride_s;
    int64_t o_stride_b, o_stride_h, o_stride_s;
    float scale;
    int32_t reserved;
    const void* q;
    const void* k;
    const void* v;
    const void* mask; /* additive [batch, seq_kv] fp16 or null */
    void* o;
} b200ml_attention_params;

/* softmax(scale * Q K^T + mask) V in one kernel, fp16 in/out, fp32 accumulate.  Replaces the
 * MatMul -> Mul -> (Add) -> Softmax -> MatMul sub-graph and the head split / merge Transposes
 * around it (pure_implementations.py:111-216, 309-326). */
int b200ml_attention_f16(b200ml_ctx* ctx, const b200ml_attention_params* p, b200ml_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* DACEML_B200_H */
