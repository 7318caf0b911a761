// extern "C" surface of libdaceml_b200: argument validation, context management, dispatch.
#include "common.cuh"
#include "tensormap.cuh"

#include <cuda.h>
#include <string.h>
#include <stdlib.h>
#include <new>

namespace b200ml {

static thread_local char g_error[512] = "";
std::atomic<int64_t> g_launches{0};

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = getenv("B200ML_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int gemm_f16(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream);
int gemm_f32(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream);
int gemm_f16_layernorm(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream);
int softmax(int dtype, const void* x, const void* mask, void* y, int64_t rows, int64_t cols, int64_t mask_row_div,
            float scale, int is_log, cudaStream_t s);
int layernorm(int dtype, const void* x, const void* residual, const void* bias, const void* gamma, const void* beta,
              void* y, int64_t rows, int64_t cols, float eps, cudaStream_t s);
int reduce(const b200ml_ctx* ctx, int dtype, int op, const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
           cudaStream_t s);
int unary(const b200ml_ctx* ctx, int dtype, int op, const void* x, void* y, int64_t n, float p0, float p1,
          cudaStream_t s);
int binary(const b200ml_ctx* ctx, int dtype, int op, const void* a, const void* b, void* y, int rank,
           const int64_t* shape, const int64_t* as, const int64_t* bs, cudaStream_t s);
int bias_act(const b200ml_ctx* ctx, int dtype, const void* x, const void* bias, const void* residual, void* y,
             int64_t rows, int64_t cols, int act, cudaStream_t s);
int transpose(const b200ml_ctx* ctx, int elem_bytes, const void* x, void* y, int rank, const int64_t* shape,
              const int32_t* perm, cudaStream_t s);
int cast(const b200ml_ctx* ctx, int src, int dst, const void* x, void* y, int64_t n, cudaStream_t s);
int cast_any(const b200ml_ctx* ctx, int src, int dst, const void* x, void* y, int64_t n, cudaStream_t s);
int conv2d(const b200ml_ctx* ctx, const b200ml_conv_params* p, cudaStream_t s);
int64_t conv_prepack_bytes(const b200ml_ctx* ctx, const b200ml_conv_params* p);
int conv_prepack(const b200ml_ctx* ctx, const b200ml_conv_params* p, void* packed, cudaStream_t s);
int se_gate(const b200ml_ctx* ctx, int dtype, const void* pooled, const void* w1, const void* b1, const void* w2,
            const void* b2, void* gate, int64_t n, int64_t c, int64_t r, cudaStream_t s);
int attention_f16(const b200ml_ctx* ctx, const b200ml_attention_params* p, cudaStream_t s);

static bool dtype_ok(int d) { return d == B200ML_F16 || d == B200ML_F32; }

// Makes the context's device current for the duration of a call when it is not already.

}  // namespace b200ml

using namespace b200ml;

#define CTX_CHECK(ctx)                                                       \
    do {                                                                     \
        if (!(ctx)) return fail(B200ML_ERR_INVALID, "%s: null context", __func__); \
    } while (0)

// ---------------------------------------------------------------------------------------------
// Tensor-map table (tensormap.cuh)
// ---------------------------------------------------------------------------------------------
namespace b200ml {
namespace {
struct TmapKey {
    uint64_t w[13];
    bool operator==(const TmapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct TmapEntry {
    TmapKey key;
    bool used = false;
    alignas(64) CUtensorMap map;
};
constexpr int kTmapSlots = 1024;  // direct-mapped; a colliding key simply replaces the older entry
thread_local TmapEntry* t_tmaps = nullptr;
thread_local int64_t t_tmap_hits = 0, t_tmap_misses = 0;
}  // namespace

CUresult encode_tiled_cached(const b200ml_ctx* ctx, CUtensorMap* out, CUtensorMapDataType dtype, const void* base,
                             const cuuint64_t dims[4], const cuuint64_t strides[3], const cuuint32_t box[4],
                             CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled);
    if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
    TmapKey key;
    key.w[0] = reinterpret_cast<uint64_t>(base);
    key.w[1] = static_cast<uint64_t>(dtype) | (static_cast<uint64_t>(swizzle) << 16) | (static_cast<uint64_t>(ctx->device) << 32);
    for (int i = 0; i < 4; ++i) key.w[2 + i] = dims[i];
    for (int i = 0; i < 3; ++i) key.w[6 + i] = strides[i];
    for (int i = 0; i < 4; ++i) key.w[9 + i] = box[i];
    uint64_t h = 1469598103934665603ull;
    for (uint64_t v : key.w) h = (h ^ v) * 1099511628211ull;
    if (!t_tmaps) t_tmaps = new (std::nothrow) TmapEntry[kTmapSlots];
    TmapEntry* e = t_tmaps ? &t_tmaps[(h >> 20) & (kTmapSlots - 1)] : nullptr;
    if (e && e->used && e->key == key) {
        ++t_tmap_hits;
        *out = e->map;
        return CUDA_SUCCESS;
    }
    ++t_tmap_misses;
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, dtype, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS && e) {
        e->key = key;
        e->map = *out;
        e->used = true;
    }
    return r;
}

void tensormap_cache_counters(int64_t* hits, int64_t* misses) {
    *hits = t_tmap_hits;
    *misses = t_tmap_misses;
}
}  // namespace b200ml

extern "C" {

int b200ml_version(void) { return 100; }

const char* b200ml_last_error(void) { return g_error; }

int64_t b200ml_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200ml_ctx_create(int device, int64_t workspace_bytes, b200ml_ctx** out) {
    B200ML_REQUIRE(out != nullptr, "ctx_create: null output pointer");
    B200ML_REQUIRE(workspace_bytes >= 0, "ctx_create: negative workspace size");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(B200ML_ERR_CUDA, "ctx_create: no CUDA device is visible (%s); this library has no CPU path",
                    cudaGetErrorString(e));
    B200ML_REQUIRE(device >= 0 && device < count, "ctx_create: device %d out of range (%d visible)", device, count);
    DeviceGuard guard(device);
    cudaDeviceProp prop;
    B200ML_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(B200ML_ERR_UNSUPPORTED, "ctx_create: device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    b200ml_ctx* ctx = new (std::nothrow) b200ml_ctx();
    if (!ctx) return fail(B200ML_ERR_CUDA, "ctx_create: out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    cudaError_t err = cudaMalloc(&ctx->status_dev, sizeof(int32_t));
    if (err == cudaSuccess) err = cudaMemset(ctx->status_dev, 0, sizeof(int32_t));
    if (err == cudaSuccess && workspace_bytes > 0) {
        err = cudaMalloc(&ctx->workspace, (size_t)workspace_bytes);
        ctx->workspace_bytes = workspace_bytes;
    }
    if (err != cudaSuccess) {
        if (ctx->status_dev) cudaFree(ctx->status_dev);
        delete ctx;
        return fail(B200ML_ERR_CUDA, "ctx_create: device allocation failed: %s", cudaGetErrorString(err));
    }
    // cuTensorMapEncodeTiled comes from the driver; resolve it through the runtime so the library
    // does not link libcuda.
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) ctx->encode_tiled = fn;
    else (void)cudaGetLastError();
    fn = nullptr;
    err = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) ctx->mem_get_address_range = fn;
    else (void)cudaGetLastError();
    *out = ctx;
    return B200ML_OK;
}

int b200ml_ctx_destroy(b200ml_ctx* ctx) {
    if (!ctx) return B200ML_OK;
    DeviceGuard guard(ctx->device);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    delete ctx;
    return B200ML_OK;
}

int b200ml_ctx_device_status(b200ml_ctx* ctx, int32_t* status) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(status != nullptr, "ctx_device_status: null output pointer");
    DeviceGuard guard(ctx->device);
    B200ML_CUDA(cudaMemcpy(status, ctx->status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (*status != 0) {
        B200ML_CUDA(cudaMemset(ctx->status_dev, 0, sizeof(int32_t)));
        return fail(B200ML_ERR_DEVICE, "%s (device status %d)",
                    *status == DEV_BAD_INDEX ? "Gather met an index outside its axis" : "a kernel gave up a bounded wait", *status);
    }
    return B200ML_OK;
}

int64_t b200ml_ctx_workspace_bytes(const b200ml_ctx* ctx) { return ctx ? ctx->workspace_bytes : 0; }

int b200ml_gemm(b200ml_ctx* ctx, const b200ml_gemm_params* p, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(p != nullptr, "gemm: null parameter block");
    B200ML_REQUIRE(dtype_ok(p->dtype), "gemm: unknown dtype %d", p->dtype);
    B200ML_REQUIRE(p->m >= 0 && p->n >= 0 && p->k >= 0, "gemm: negative extent");
    B200ML_REQUIRE(p->batch_outer >= 1 && p->batch_inner >= 1, "gemm: batch extents must be >= 1");
    B200ML_REQUIRE(p->m < (1ll << 31) && p->n < (1ll << 31) && p->k < (1ll << 31), "gemm: extent too large");
    if (p->m == 0 || p->n == 0) return B200ML_OK;
    B200ML_REQUIRE(p->k > 0, "gemm: empty reduction extent");
    B200ML_REQUIRE(p->a && p->b && p->c, "gemm: null operand");
    B200ML_REQUIRE(!(p->epilogue & B200ML_EPI_BIAS) || p->bias, "gemm: bias epilogue without a bias pointer");
    B200ML_REQUIRE(!(p->epilogue & B200ML_EPI_RESIDUAL) || p->residual, "gemm: residual epilogue without a residual pointer");
    B200ML_REQUIRE(p->a_layout == 0 || p->a_layout == 1, "gemm: bad a_layout");
    B200ML_REQUIRE(p->b_layout == 0 || p->b_layout == 1, "gemm: bad b_layout");
    B200ML_REQUIRE(p->lda >= (p->a_layout ? p->m : p->k), "gemm: lda too small");
    B200ML_REQUIRE(p->ldb >= (p->b_layout ? p->k : p->n), "gemm: ldb too small");
    B200ML_REQUIRE(p->ldc >= p->n, "gemm: ldc too small");
    DeviceGuard guard(ctx->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (p->epilogue & B200ML_EPI_LAYERNORM) {
        if (p->dtype != B200ML_F16) return fail(B200ML_ERR_UNSUPPORTED, "gemm + layernorm: fp16 only");
        return gemm_f16_layernorm(ctx, p, s);
    }
    return p->dtype == B200ML_F16 ? gemm_f16(ctx, p, s) : gemm_f32(ctx, p, s);
}

int b200ml_softmax(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* mask, void* y, int64_t rows,
                   int64_t cols, int64_t mask_row_div, float scale, int32_t is_log, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "softmax: unknown dtype %d", dtype);
    B200ML_REQUIRE(rows >= 0 && cols >= 0, "softmax: negative extent");
    if (rows == 0 || cols == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "softmax: null tensor");
    B200ML_REQUIRE(cols < (1ll << 31), "softmax: row too long");
    B200ML_REQUIRE(!mask || mask_row_div >= 1, "softmax: mask_row_div must be >= 1");
    DeviceGuard guard(ctx->device);
    return softmax(dtype, x, mask, y, rows, cols, mask ? mask_row_div : 1, scale, is_log, static_cast<cudaStream_t>(stream));
}

int b200ml_layernorm(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* residual, const void* bias,
                     const void* gamma, const void* beta, void* y, int64_t rows, int64_t cols, float eps,
                     b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "layernorm: unknown dtype %d", dtype);
    B200ML_REQUIRE(rows >= 0 && cols >= 0, "layernorm: negative extent");
    if (rows == 0 || cols == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "layernorm: null tensor");
    B200ML_REQUIRE(cols < (1ll << 31), "layernorm: row too long");
    DeviceGuard guard(ctx->device);
    return layernorm(dtype, x, residual, bias, gamma, beta, y, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int b200ml_reduce(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* x, void* y, int64_t outer, int64_t red,
                  int64_t inner, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "reduce: unknown dtype %d", dtype);
    B200ML_REQUIRE(op >= B200ML_RED_SUM && op <= B200ML_RED_MIN, "reduce: unknown op %d", op);
    B200ML_REQUIRE(outer >= 0 && red >= 0 && inner >= 0, "reduce: negative extent");
    if (outer == 0 || inner == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "reduce: null tensor");
    DeviceGuard guard(ctx->device);
    return reduce(ctx, dtype, op, x, y, outer, red, inner, static_cast<cudaStream_t>(stream));
}

int b200ml_unary(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* x, void* y, int64_t n, float p0, float p1,
                 b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "unary: unknown dtype %d", dtype);
    B200ML_REQUIRE(op >= B200ML_UN_COPY && op <= B200ML_UN_ABS, "unary: unknown op %d", op);
    B200ML_REQUIRE(n >= 0, "unary: negative extent");
    if (n == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "unary: null tensor");
    DeviceGuard guard(ctx->device);
    return unary(ctx, dtype, op, x, y, n, p0, p1, static_cast<cudaStream_t>(stream));
}

int b200ml_binary(b200ml_ctx* ctx, int32_t dtype, int32_t op, const void* a, const void* b, void* y, int32_t rank,
                  const int64_t* shape, const int64_t* a_strides, const int64_t* b_strides, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "binary: unknown dtype %d", dtype);
    B200ML_REQUIRE(op >= B200ML_BIN_ADD && op <= B200ML_BIN_MIN, "binary: unknown op %d", op);
    B200ML_REQUIRE(rank >= 0 && rank <= 6, "binary: rank %d not in [0, 6]", rank);
    B200ML_REQUIRE(rank == 0 || (shape && a_strides && b_strides), "binary: null shape or strides");
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] >= 0, "binary: negative extent");
        if (shape[d] == 0) return B200ML_OK;
    }
    B200ML_REQUIRE(a && b && y, "binary: null tensor");
    DeviceGuard guard(ctx->device);
    return binary(ctx, dtype, op, a, b, y, rank, shape, a_strides, b_strides, static_cast<cudaStream_t>(stream));
}

int b200ml_bias_act(b200ml_ctx* ctx, int32_t dtype, const void* x, const void* bias, const void* residual, void* y,
                    int64_t rows, int64_t cols, int32_t act, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "bias_act: unknown dtype %d", dtype);
    B200ML_REQUIRE(rows >= 0 && cols >= 0, "bias_act: negative extent");
    if (rows == 0 || cols == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "bias_act: null tensor");
    DeviceGuard guard(ctx->device);
    return bias_act(ctx, dtype, x, bias, residual, y, rows, cols, act, static_cast<cudaStream_t>(stream));
}

int b200ml_transpose(b200ml_ctx* ctx, int32_t elem_bytes, const void* x, void* y, int32_t rank, const int64_t* shape,
                     const int32_t* perm, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(elem_bytes == 2 || elem_bytes == 4, "transpose: element size %d not supported", elem_bytes);
    B200ML_REQUIRE(rank >= 1 && rank <= 6, "transpose: rank %d not in [1, 6]", rank);
    B200ML_REQUIRE(shape && perm, "transpose: null shape or perm");
    uint32_t seen = 0;
    for (int d = 0; d < rank; ++d) {
        B200ML_REQUIRE(shape[d] >= 0, "transpose: negative extent");
        B200ML_REQUIRE(perm[d] >= 0 && perm[d] < rank && !(seen & (1u << perm[d])), "transpose: perm is not a permutation");
        seen |= 1u << perm[d];
    }
    for (int d = 0; d < rank; ++d)
        if (shape[d] == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "transpose: null tensor");
    DeviceGuard guard(ctx->device);
    return transpose(ctx, elem_bytes, x, y, rank, shape, perm, static_cast<cudaStream_t>(stream));
}

int b200ml_cast(b200ml_ctx* ctx, int32_t src_dtype, int32_t dst_dtype, const void* x, void* y, int64_t n,
                b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(src_dtype >= B200ML_F16 && src_dtype <= B200ML_BOOL && dst_dtype >= B200ML_F16 && dst_dtype <= B200ML_BOOL,
                   "cast: unknown dtype");
    B200ML_REQUIRE(n >= 0, "cast: negative extent");
    if (n == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "cast: null tensor");
    DeviceGuard guard(ctx->device);
    if (dtype_ok(src_dtype) && dtype_ok(dst_dtype))
        return cast(ctx, src_dtype, dst_dtype, x, y, n, static_cast<cudaStream_t>(stream));
    return cast_any(ctx, src_dtype, dst_dtype, x, y, n, static_cast<cudaStream_t>(stream));
}

int64_t b200ml_conv_prepack_bytes(b200ml_ctx* ctx, const b200ml_conv_params* p) {
    if (ctx == nullptr || p == nullptr || p->dtype != B200ML_F32) return 0;
    return conv_prepack_bytes(ctx, p);
}

int b200ml_conv_prepack(b200ml_ctx* ctx, const b200ml_conv_params* p, void* packed, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(p != nullptr, "conv_prepack: null parameter block");
    return conv_prepack(ctx, p, packed, static_cast<cudaStream_t>(stream));
}

int b200ml_conv2d(b200ml_ctx* ctx, const b200ml_conv_params* p, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(p != nullptr, "conv: null parameter block");
    B200ML_REQUIRE(dtype_ok(p->dtype), "conv: unknown dtype %d", p->dtype);
    B200ML_REQUIRE(p->n >= 0 && p->c >= 1 && p->h >= 1 && p->w >= 1 && p->m >= 0, "conv: bad tensor extent");
    B200ML_REQUIRE(p->pad_top >= 0 && p->pad_left >= 0 && p->pad_bottom >= 0 && p->pad_right >= 0, "conv: negative pad");
    B200ML_REQUIRE(p->n * p->c * p->h * p->w < (1ll << 40), "conv: input too large");
    B200ML_REQUIRE(p->h < (1 << 24) && p->w < (1 << 24) && p->c < (1 << 24) && p->m < (1 << 24) && p->n < (1 << 24),
                   "conv: extent too large");
    if (p->n == 0 || p->m == 0) return B200ML_OK;
    B200ML_REQUIRE(p->x && p->weight && p->y, "conv: null tensor");
    DeviceGuard guard(ctx->device);
    return conv2d(ctx, p, static_cast<cudaStream_t>(stream));
}

int b200ml_se_gate(b200ml_ctx* ctx, int32_t dtype, const void* pooled, const void* w1, const void* b1, const void* w2,
                   const void* b2, void* gate, int64_t n, int64_t c, int64_t r, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(dtype_ok(dtype), "se_gate: unknown dtype %d", dtype);
    B200ML_REQUIRE(n >= 0 && c >= 0 && r >= 1, "se_gate: bad extent");
    if (n == 0 || c == 0) return B200ML_OK;
    B200ML_REQUIRE(pooled && w1 && w2 && gate, "se_gate: null tensor");
    B200ML_REQUIRE(n < (1ll << 31), "se_gate: too many images");
    DeviceGuard guard(ctx->device);
    return se_gate(ctx, dtype, pooled, w1, b1, w2, b2, gate, n, c, r, static_cast<cudaStream_t>(stream));
}

int b200ml_attention_f16(b200ml_ctx* ctx, const b200ml_attention_params* p, b200ml_stream stream) {
    CTX_CHECK(ctx);
    B200ML_REQUIRE(p != nullptr, "attention: null parameter block");
    B200ML_REQUIRE(p->batch >= 0 && p->heads >= 0 && p->seq_q >= 0 && p->seq_kv >= 0 && p->head_dim >= 1,
                   "attention: bad extent");
    if (p->batch == 0 || p->heads == 0 || p->seq_q == 0) return B200ML_OK;
    B200ML_REQUIRE(p->seq_kv > 0, "attention: empty key sequence");
    B200ML_REQUIRE(p->q && p->k && p->v && p->o, "attention: null tensor");
    DeviceGuard guard(ctx->device);
    return attention_f16(ctx, p, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
