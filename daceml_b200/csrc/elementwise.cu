// Element-wise operators: unary maps, numpy-broadcast binary maps, bias + activation (+ residual),
// permutations and casts.  Contiguous cases move 16 bytes per thread per access; math is fp32.
#include "common.cuh"
#include "epilogue.cuh"

namespace b200ml {

namespace {

__device__ __forceinline__ float ldf(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldf(const __half* p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__half* p, float v) { *p = __float2half_rn(v); }

template <typename T>
struct Pack;
template <>
struct Pack<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half* p, float (&f)[8]) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(p)), f);
    }
    static __device__ __forceinline__ void store(__half* p, const float (&f)[8]) {
        *reinterpret_cast<uint4*>(p) = pack8(f);
    }
};
template <>
struct Pack<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(p));
        f[0] = q.x, f[1] = q.y, f[2] = q.z, f[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
};

__device__ __forceinline__ float unary_apply(int op, float x, float p0, float p1) {
    switch (op) {
        case B200ML_UN_COPY: return x;
        case B200ML_UN_RELU: return fmaxf(x, 0.0f);
        case B200ML_UN_SIGMOID: return sigmoidf_(x);
        case B200ML_UN_ERF: return erff(x);
        case B200ML_UN_SQRT: return sqrtf(x);
        case B200ML_UN_EXP: return expf(x);
        case B200ML_UN_LOG: return logf(x);
        case B200ML_UN_TANH: return tanhf(x);
        case B200ML_UN_SWISH: return x * sigmoidf_(x);
        case B200ML_UN_GELU: return gelu_erf(x);
        case B200ML_UN_RECIPROCAL: return 1.0f / x;
        case B200ML_UN_LEAKYRELU: return fmaxf(x, 0.0f) + p0 * fminf(x, 0.0f);
        case B200ML_UN_AFFINE: return fmaf(p0, x, p1);
        case B200ML_UN_POWS: return p0 == 2.0f ? x * x : powf(x, p0);
        case B200ML_UN_SOFTPLUS: return log1pf(expf(x));
        case B200ML_UN_CLIP: return fminf(fmaxf(x, p0), p1);
        case B200ML_UN_NEG: return -x;
        case B200ML_UN_ABS: return fabsf(x);
        default: return x;
    }
}

__device__ __forceinline__ float binary_apply(int op, float a, float b) {
    switch (op) {
        case B200ML_BIN_ADD: return a + b;
        case B200ML_BIN_SUB: return a - b;
        case B200ML_BIN_MUL: return a * b;
        case B200ML_BIN_DIV: return a / b;
        case B200ML_BIN_POW: return b == 2.0f ? a * a : powf(a, b);
        case B200ML_BIN_MAX: return fmaxf(a, b);
        case B200ML_BIN_MIN: return fminf(a, b);
        default: return a;
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) unary_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, int op,
                                                    float p0, float p1) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = VEC ? Pack<T>::N : 1;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += stride) {
        if (VEC) {
            float f[Pack<T>::N];
            Pack<T>::load(x + i, f);
#pragma unroll
            for (int j = 0; j < Pack<T>::N; ++j)
                f[j] = (sizeof(T) == 2 && op == B200ML_UN_GELU) ? gelu_erf_fast(f[j]) : unary_apply(op, f[j], p0, p1);
            Pack<T>::store(y + i, f);
        } else {
            stf(y + i, unary_apply(op, ldf(x + i), p0, p1));
        }
    }
}

// The vector form of the unary map with the operator fixed at compile time and two packets per thread and step.
template <typename T, int OP>
__global__ void __launch_bounds__(256) unary2_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t n, float p0, float p1) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = Pack<T>::N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += 2 * stride) {
        const int64_t i2 = i + stride;
        const bool second = i2 < n;
        float f[V], g[V];
        Pack<T>::load(x + i, f);
        if (second) Pack<T>::load(x + i2, g);
#pragma unroll
        for (int j = 0; j < V; ++j) f[j] = unary_apply(OP, f[j], p0, p1);
        Pack<T>::store(y + i, f);
        if (second) {
#pragma unroll
            for (int j = 0; j < V; ++j) g[j] = unary_apply(OP, g[j], p0, p1);
            Pack<T>::store(y + i2, g);
        }
    }
}

// Same-shape contiguous operands (mode 0), b a scalar (mode 1), or b a vector along the last
// axis of length period (mode 2, the bias pattern).
template <typename T>
__global__ void __launch_bounds__(256) binary_fast_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          T* __restrict__ y, int64_t n, int op, int mode,
                                                          int64_t period, int swap) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = Pack<T>::N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    const float bs = mode == 1 ? ldf(b) : 0.0f;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    int64_t col = mode == 2 ? first % period : 0;  // one 64-bit remainder per thread, not per packet
    const int64_t col_step = mode == 2 ? stride % period : 0;
    for (int64_t i = first; i < n; i += stride) {
        float fa[V], fb[V];
        Pack<T>::load(a + i, fa);
        if (mode == 0) Pack<T>::load(b + i, fb);
        else if (mode == 2) {
            Pack<T>::load(b + col, fb);
            col += col_step;
            if (col >= period) col -= period;
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const float bv = mode == 1 ? bs : fb[j];
            fa[j] = swap ? binary_apply(op, bv, fa[j]) : binary_apply(op, fa[j], bv);
        }
        Pack<T>::store(y + i, fa);
    }
}

// Same-shape contiguous operands, operator fixed at compile time (no branch in the loop), two packets per thread and
// step so that four 16-byte loads are in flight before the first result is needed.
template <typename T, int OP>
__global__ void __launch_bounds__(256) binary_same_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                          T* __restrict__ y, int64_t n) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = Pack<T>::N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V; i < n; i += 2 * stride) {
        const int64_t i2 = i + stride;
        const bool second = i2 < n;
        float fa[V], fb[V], ga[V], gb[V];
        Pack<T>::load(a + i, fa);
        Pack<T>::load(b + i, fb);
        if (second) {
            Pack<T>::load(a + i2, ga);
            Pack<T>::load(b + i2, gb);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) fa[j] = binary_apply(OP, fa[j], fb[j]);
        Pack<T>::store(y + i, fa);
        if (second) {
#pragma unroll
            for (int j = 0; j < V; ++j) ga[j] = binary_apply(OP, ga[j], gb[j]);
            Pack<T>::store(y + i2, ga);
        }
    }
}

struct BcastArgs {
    int32_t rank;
    int64_t shape[6];
    int64_t as[6];
    int64_t bs[6];
};

template <typename T>
__global__ void __launch_bounds__(256) binary_bcast_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                           T* __restrict__ y, int64_t n, int op, const BcastArgs g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, ao = 0, bo = 0;
#pragma unroll
        for (int d = 5; d >= 0; --d) {
            if (d < g.rank) {
                const int64_t c = rem % g.shape[d];
                rem /= g.shape[d];
                ao += c * g.as[d];
                bo += c * g.bs[d];
            }
        }
        stf(y + i, binary_apply(op, ldf(a + ao), ldf(b + bo)));
    }
}

template <typename T>
__device__ __forceinline__ float act_for(float v, int act) { return apply_act(v, act); }
template <>
__device__ __forceinline__ float act_for<__half>(float v, int act) { return apply_act_f16(v, act); }

__device__ __forceinline__ void gelu_store8(__half* y, float (&f)[8], const float (&b)[8], bool has_bias) {
    if (has_bias) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += b[j];
    }
    *reinterpret_cast<uint4*>(y) = gelu_pack8(f);
}
__device__ __forceinline__ void gelu_store8(float*, float (&)[4], const float (&)[4], bool) {}  // never taken: fp32 keeps fp32 math

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                                       const T* __restrict__ residual, T* __restrict__ y, int64_t n,
                                                       int64_t cols, int act) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = VEC ? Pack<T>::N : 1;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    int64_t col = VEC ? first % cols : 0;  // the bias column advances by (stride mod cols): one 64-bit remainder per thread
    const int64_t col_step = VEC ? stride % cols : 0;
    const bool half_gelu = VEC && sizeof(T) == 2 && act == B200ML_EPI_GELU && !residual;
    for (int64_t i = first; i < n; i += stride) {
        if (VEC) {
            float f[Pack<T>::N], t[Pack<T>::N];
            Pack<T>::load(x + i, f);
            if (bias) {
                Pack<T>::load(bias + col, t);
                col += col_step;
                if (col >= cols) col -= cols;
            }
            if (half_gelu) {  // fp16 bias + GELU: pairs in half precision, half the instructions per value
                gelu_store8(y + i, f, t, bias != nullptr);
                continue;
            }
            if (bias) {
#pragma unroll
                for (int j = 0; j < Pack<T>::N; ++j) f[j] += t[j];
            }
#pragma unroll
            for (int j = 0; j < Pack<T>::N; ++j) f[j] = act_for<T>(f[j], act);
            if (residual) {
                Pack<T>::load(residual + i, t);
#pragma unroll
                for (int j = 0; j < Pack<T>::N; ++j) f[j] += t[j];
            }
            Pack<T>::store(y + i, f);
        } else {
            float v = ldf(x + i) + (bias ? ldf(bias + i % cols) : 0.0f);
            v = act_for<T>(v, act);
            if (residual) v += ldf(residual + i);
            stf(y + i, v);
        }
    }
}

// The vector form with the activation fixed at compile time and two packets per thread and step: every 16-byte load of
// both packets is issued before the first activation is evaluated.
template <typename T, int ACT>
__global__ void __launch_bounds__(256) bias_act2_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                                        const T* __restrict__ residual, T* __restrict__ y, int64_t n,
                                                        int64_t cols) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = Pack<T>::N;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * V;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * V;
    // the bias column of a packet advances by (stride mod cols) per step: one 64-bit remainder per thread, not per packet
    int64_t col = first % cols;
    const int64_t col_step = stride % cols;
    for (int64_t i = first; i < n; i += 2 * stride) {
        const int64_t idx[2] = {i, i + stride};
        const bool on[2] = {true, i + stride < n};
        int64_t cols_of[2];
        cols_of[0] = col;
        col += col_step;
        if (col >= cols) col -= cols;
        cols_of[1] = col;
        col += col_step;
        if (col >= cols) col -= cols;
        float f[2][V], r[2][V], b[2][V];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!on[u]) continue;
            Pack<T>::load(x + idx[u], f[u]);
            if (residual) Pack<T>::load(residual + idx[u], r[u]);
            if (bias) Pack<T>::load(bias + cols_of[u], b[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!on[u]) continue;
            if (ACT == B200ML_EPI_GELU && sizeof(T) == 2 && !residual) {  // fp16 bias + GELU: pairs in half precision
                gelu_store8(y + idx[u], f[u], b[u], bias != nullptr);
                continue;
            }
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float v = f[u][j] + (bias ? b[u][j] : 0.0f);
                v = act_for<T>(v, ACT);
                f[u][j] = residual ? v + r[u][j] : v;
            }
            Pack<T>::store(y + idx[u], f[u]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Permutation.  The output is walked linearly; when the innermost output axis is not the
// innermost input axis, a 32x32 shared-memory tile turns strided reads into coalesced ones.
// ---------------------------------------------------------------------------------------------
struct PermArgs {
    int32_t rank;
    int64_t oshape[6];   // output shape
    int64_t istride[6];  // input element stride of each output axis
};

template <typename E>
__global__ void __launch_bounds__(256) permute_gather_kernel(const E* __restrict__ x, E* __restrict__ y, int64_t n,
                                                             const PermArgs g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, off = 0;
#pragma unroll
        for (int d = 5; d >= 0; --d) {
            if (d < g.rank) {
                off += (rem % g.oshape[d]) * g.istride[d];
                rem /= g.oshape[d];
            }
        }
        y[i] = x[off];
    }
}

// Batched 2-D transpose: y[b][j][i] = x at (b, i, j) where i is the input's contiguous axis seen
// from the output (stride 1 in the input) and j is the output's contiguous axis.
// Batch offsets are decoded from the remaining output axes.
struct TileArgs {
    int32_t rank;        // rank of the batch index space
    int64_t bshape[6];   // batch extents (output order, without the two tiled axes)
    int64_t bistride[6]; // input strides of the batch axes
    int64_t bostride[6]; // output strides of the batch axes
    int64_t ni, nj;      // extents of i (input-contiguous) and j (output-contiguous)
    int64_t j_istride;   // input stride of j
    int64_t i_ostride;   // output stride of i
};

template <typename E>
__global__ void __launch_bounds__(256) permute_tiled_kernel(const E* __restrict__ x, E* __restrict__ y,
                                                            const TileArgs g) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    __shared__ E tile[32][33];
    int64_t b = blockIdx.z, ioff = 0, ooff = 0;
#pragma unroll
    for (int d = 5; d >= 0; --d) {
        if (d < g.rank) {
            const int64_t c = b % g.bshape[d];
            b /= g.bshape[d];
            ioff += c * g.bistride[d];
            ooff += c * g.bostride[d];
        }
    }
    const int64_t i0 = static_cast<int64_t>(blockIdx.x) * 32, j0 = static_cast<int64_t>(blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int r = 0; r < 32; r += 8) {
        const int64_t i = i0 + tx, j = j0 + ty + r;
        if (i < g.ni && j < g.nj) tile[ty + r][tx] = x[ioff + j * g.j_istride + i];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 32; r += 8) {
        const int64_t j = j0 + tx, i = i0 + ty + r;
        if (i < g.ni && j < g.nj) y[ooff + i * g.i_ostride + j] = tile[tx][ty + r];
    }
}

template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_kernel(const S* __restrict__ x, D* __restrict__ y, int64_t n) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        stf(y + i, ldf(x + i));
}

inline unsigned grid_for(int64_t work_items, int sms) {
    int64_t blocks = ceil_div(work_items, 256);
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<unsigned>(blocks);
}

template <typename T>
int unary_t(const b200ml_ctx* ctx, int op, const T* x, T* y, int64_t n, float p0, float p1, cudaStream_t s) {
    constexpr int V = Pack<T>::N;
    if (n % V == 0 && aligned16(x) && aligned16(y)) {
        const unsigned grid = grid_for((n / V + 1) / 2, ctx->sm_count);
#define B200ML_UNARY2(OP) case OP: launch_pdl(unary2_kernel<T, OP>, dim3(grid), dim3(256), 0, s, x, y, n, p0, p1); break
        switch (op) {  // the load-bound operators; those bound by instruction issue (GELU, Swish, ...) gain nothing from it
            B200ML_UNARY2(B200ML_UN_COPY);
            B200ML_UNARY2(B200ML_UN_RELU);
            B200ML_UNARY2(B200ML_UN_AFFINE);
            B200ML_UNARY2(B200ML_UN_CLIP);
            B200ML_UNARY2(B200ML_UN_NEG);
            default: launch_pdl(unary_kernel<T, true>, dim3(grid_for(n / V, ctx->sm_count)), dim3(256), 0, s, x, y, n, op, p0, p1); break;
        }
#undef B200ML_UNARY2
    } else {
        launch_pdl(unary_kernel<T, false>, dim3(grid_for(n, ctx->sm_count)), dim3(256), 0, s, x, y, n, op, p0, p1);
    }
    return check_launch("unary");
}

template <typename T>
int binary_t(const b200ml_ctx* ctx, int op, const T* a, const T* b, T* y, int rank, const int64_t* shape,
             const int64_t* as, const int64_t* bs, cudaStream_t s) {
    constexpr int V = Pack<T>::N;
    int64_t n = 1;
    for (int d = 0; d < rank; ++d) n *= shape[d];
    if (n == 0) return B200ML_OK;
    // Classify each operand: dense (contiguous strides), scalar (all zero), or a vector on the
    // last axis (stride 1 there, zero elsewhere).
    auto classify = [&](const int64_t* st) {
        bool dense = true, scalar = true, lastvec = rank >= 1;
        int64_t expect = 1;
        for (int d = rank - 1; d >= 0; --d) {
            if (shape[d] != 1) {
                if (st[d] != expect) dense = false;
                if (st[d] != 0) scalar = false;
                if (d == rank - 1 ? st[d] != 1 : st[d] != 0) lastvec = false;
            }
            expect *= shape[d];
        }
        return dense ? 0 : (scalar ? 1 : (lastvec ? 2 : 3));
    };
    const int ca = rank == 0 ? 0 : classify(as), cb = rank == 0 ? 0 : classify(bs);
    const int64_t last = rank ? shape[rank - 1] : 1;
    const bool vec_ok = n % V == 0 && aligned16(y);
    if (vec_ok && ca == 0 && cb == 0 && aligned16(a) && aligned16(b) && op <= B200ML_BIN_DIV) {
        const unsigned grid = grid_for((n / V + 1) / 2, ctx->sm_count);
        switch (op) {
            case B200ML_BIN_ADD: launch_pdl(binary_same_kernel<T, B200ML_BIN_ADD>, dim3(grid), dim3(256), 0, s, a, b, y, n); break;
            case B200ML_BIN_SUB: launch_pdl(binary_same_kernel<T, B200ML_BIN_SUB>, dim3(grid), dim3(256), 0, s, a, b, y, n); break;
            case B200ML_BIN_MUL: launch_pdl(binary_same_kernel<T, B200ML_BIN_MUL>, dim3(grid), dim3(256), 0, s, a, b, y, n); break;
            default: launch_pdl(binary_same_kernel<T, B200ML_BIN_DIV>, dim3(grid), dim3(256), 0, s, a, b, y, n); break;
        }
        return check_launch("binary_same");
    }
    if (vec_ok && ca == 0 && aligned16(a) && (cb == 0 ? aligned16(b) : cb == 1 ? true : (cb == 2 && last % V == 0 && aligned16(b)))) {
        launch_pdl(binary_fast_kernel<T>, dim3(grid_for(n / V, ctx->sm_count)), dim3(256), 0, s, a, b, y, n, op, cb, last, 0);
        return check_launch("binary_fast");
    }
    if (vec_ok && cb == 0 && aligned16(b) && (ca == 1 || (ca == 2 && last % V == 0 && aligned16(a)))) {
        launch_pdl(binary_fast_kernel<T>, dim3(grid_for(n / V, ctx->sm_count)), dim3(256), 0, s, b, a, y, n, op, ca, last, 1);
        return check_launch("binary_fast");
    }
    BcastArgs g{};
    g.rank = rank;
    for (int d = 0; d < rank; ++d) {
        g.shape[d] = shape[d];
        g.as[d] = shape[d] == 1 ? 0 : as[d];
        g.bs[d] = shape[d] == 1 ? 0 : bs[d];
    }
    launch_pdl(binary_bcast_kernel<T>, dim3(grid_for(n, ctx->sm_count)), dim3(256), 0, s, a, b, y, n, op, g);
    return check_launch("binary_bcast");
}

template <typename T>
int bias_act_t(const b200ml_ctx* ctx, const T* x, const T* bias, const T* residual, T* y, int64_t rows, int64_t cols,
               int act, cudaStream_t s) {
    constexpr int V = Pack<T>::N;
    const int64_t n = rows * cols;
    if (n == 0) return B200ML_OK;
    const bool vec = cols % V == 0 && aligned16(x) && aligned16(y) && (!bias || aligned16(bias)) &&
                     (!residual || aligned16(residual));
    if (vec) {
        const unsigned grid = grid_for((n / V + 1) / 2, ctx->sm_count);
        switch (act) {
            case 0: launch_pdl(bias_act2_kernel<T, 0>, dim3(grid), dim3(256), 0, s, x, bias, residual, y, n, cols); break;
            case B200ML_EPI_RELU: launch_pdl(bias_act2_kernel<T, B200ML_EPI_RELU>, dim3(grid), dim3(256), 0, s, x, bias, residual, y, n, cols); break;
            // GELU and Swish are bound by instruction issue, not by loads: two packets per thread made them slower
            // (measured twice), so they keep one packet per thread; fp16 GELU runs on half2 pairs inside it
            default: launch_pdl(bias_act_kernel<T, true>, dim3(grid_for(n / V, ctx->sm_count)), dim3(256), 0, s, x, bias, residual, y, n, cols, act); break;
        }
    }
    else launch_pdl(bias_act_kernel<T, false>, dim3(grid_for(n, ctx->sm_count)), dim3(256), 0, s, x, bias, residual, y, n, cols, act);
    return check_launch("bias_act");
}

template <typename E>
int transpose_t(const b200ml_ctx* ctx, const E* x, E* y, int rank, const int64_t* shape, const int32_t* perm,
                cudaStream_t s) {
    int64_t istr[6], n = 1;
    {
        int64_t acc = 1;
        for (int d = rank - 1; d >= 0; --d) {
            istr[d] = acc;
            acc *= shape[d];
        }
        n = acc;
    }
    if (n == 0) return B200ML_OK;
    // Output axes with their input strides; drop size-1 axes and merge axes that stay adjacent.
    int64_t osh[6], ois[6];
    int r = 0;
    for (int d = 0; d < rank; ++d) {
        const int64_t ext = shape[perm[d]];
        if (ext == 1) continue;
        if (r > 0 && ois[r - 1] == ext * istr[perm[d]]) {
            osh[r - 1] *= ext;
            ois[r - 1] = istr[perm[d]];
        } else {
            osh[r] = ext;
            ois[r] = istr[perm[d]];
            ++r;
        }
    }
    if (r == 0) {
        osh[0] = 1;
        ois[0] = 1;
        r = 1;
    }
    if (r == 1 && ois[0] == 1) {
        B200ML_CUDA(cudaMemcpyAsync(y, x, n * sizeof(E), cudaMemcpyDeviceToDevice, s));
        count_launch();
        return B200ML_OK;
    }
    // Find the output axis that is contiguous in the input.
    int ci = -1;
    for (int d = 0; d < r; ++d)
        if (ois[d] == 1) ci = d;
    if (ci >= 0 && ci != r - 1 && osh[ci] >= 8 && osh[r - 1] >= 8) {
        TileArgs g{};
        int64_t ostr[6], acc = 1;
        for (int d = r - 1; d >= 0; --d) {
            ostr[d] = acc;
            acc *= osh[d];
        }
        int br = 0;
        int64_t batches = 1;
        for (int d = 0; d < r - 1; ++d) {
            if (d == ci) continue;
            g.bshape[br] = osh[d];
            g.bistride[br] = ois[d];
            g.bostride[br] = ostr[d];
            batches *= osh[d];
            ++br;
        }
        g.rank = br;
        g.ni = osh[ci];
        g.nj = osh[r - 1];
        g.j_istride = ois[r - 1];
        g.i_ostride = ostr[ci];
        const int64_t gx = ceil_div(g.ni, 32), gy = ceil_div(g.nj, 32);
        if (gy <= 65535 && batches <= 65535) {
            launch_pdl(permute_tiled_kernel<E>, dim3(dim3((unsigned)gx, (unsigned)gy, (unsigned)batches)), dim3(256), 0, s, x, y, g);
            return check_launch("permute_tiled");
        }
    }
    PermArgs g{};
    g.rank = r;
    for (int d = 0; d < r; ++d) {
        g.oshape[d] = osh[d];
        g.istride[d] = ois[d];
    }
    launch_pdl(permute_gather_kernel<E>, dim3(grid_for(n, ctx->sm_count)), dim3(256), 0, s, x, y, n, g);
    return check_launch("permute_gather");
}

}  // namespace

int unary(const b200ml_ctx* ctx, int dtype, int op, const void* x, void* y, int64_t n, float p0, float p1,
          cudaStream_t s) {
    if (n == 0) return B200ML_OK;
    if (dtype == B200ML_F16) return unary_t<__half>(ctx, op, (const __half*)x, (__half*)y, n, p0, p1, s);
    return unary_t<float>(ctx, op, (const float*)x, (float*)y, n, p0, p1, s);
}

int binary(const b200ml_ctx* ctx, int dtype, int op, const void* a, const void* b, void* y, int rank,
           const int64_t* shape, const int64_t* as, const int64_t* bs, cudaStream_t s) {
    if (dtype == B200ML_F16)
        return binary_t<__half>(ctx, op, (const __half*)a, (const __half*)b, (__half*)y, rank, shape, as, bs, s);
    return binary_t<float>(ctx, op, (const float*)a, (const float*)b, (float*)y, rank, shape, as, bs, s);
}

int bias_act(const b200ml_ctx* ctx, int dtype, const void* x, const void* bias, const void* residual, void* y,
             int64_t rows, int64_t cols, int act, cudaStream_t s) {
    if (dtype == B200ML_F16)
        return bias_act_t<__half>(ctx, (const __half*)x, (const __half*)bias, (const __half*)residual, (__half*)y, rows,
                                  cols, act, s);
    return bias_act_t<float>(ctx, (const float*)x, (const float*)bias, (const float*)residual, (float*)y, rows, cols,
                             act, s);
}

int transpose(const b200ml_ctx* ctx, int elem_bytes, const void* x, void* y, int rank, const int64_t* shape,
              const int32_t* perm, cudaStream_t s) {
    // The innermost axis stays innermost (the head split / merge of attention, [B,S,h,d] <-> [B,h,S,d]) and its rows are
    // whole 16-byte packets: permute packets, not elements.
    if (rank >= 2 && rank <= 6 && perm[rank - 1] == rank - 1 && (shape[rank - 1] * elem_bytes) % 16 == 0 && aligned16(x) && aligned16(y)) {
        int64_t packed[6];
        for (int d = 0; d < rank; ++d) packed[d] = shape[d];
        packed[rank - 1] = shape[rank - 1] * elem_bytes / 16;
        return transpose_t<uint4>(ctx, (const uint4*)x, (uint4*)y, rank, packed, perm, s);
    }
    if (elem_bytes == 2) return transpose_t<uint16_t>(ctx, (const uint16_t*)x, (uint16_t*)y, rank, shape, perm, s);
    return transpose_t<uint32_t>(ctx, (const uint32_t*)x, (uint32_t*)y, rank, shape, perm, s);
}

int cast(const b200ml_ctx* ctx, int src, int dst, const void* x, void* y, int64_t n, cudaStream_t s) {
    if (n == 0) return B200ML_OK;
    const unsigned grid = grid_for(n, ctx->sm_count);
    if (src == B200ML_F16 && dst == B200ML_F32) launch_pdl(cast_kernel<__half, float>, dim3(grid), dim3(256), 0, s, (const __half*)x, (float*)y, n);
    else if (src == B200ML_F32 && dst == B200ML_F16) launch_pdl(cast_kernel<float, __half>, dim3(grid), dim3(256), 0, s, (const float*)x, (__half*)y, n);
    else if (src == B200ML_F32) launch_pdl(cast_kernel<float, float>, dim3(grid), dim3(256), 0, s, (const float*)x, (float*)y, n);
    else launch_pdl(cast_kernel<__half, __half>, dim3(grid), dim3(256), 0, s, (const __half*)x, (__half*)y, n);
    return check_launch("cast");
}

}  // namespace b200ml
