// Bandwidth-bound row kernels: (scale + mask +) Softmax / LogSoftmax, (residual + bias +) LayerNorm
// and the Reduce* family.  A row lives in one warp's registers whenever it fits: 128-bit coalesced
// loads, fp32 math, warp-shuffle reductions, one read and one write of HBM per element.
#include "common.cuh"
#include "epilogue.cuh"
#include <float.h>
#include <atomic>

namespace b200ml {

namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}

// A 16-byte packet of T: 8 halves or 4 floats.
template <typename T>
struct Vec;
template <>
struct Vec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half* p, float (&f)[8]) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(p)), f);
    }
    static __device__ __forceinline__ void store(__half* p, const float (&f)[8]) {
        *reinterpret_cast<uint4*>(p) = pack8(f);
    }
};
template <>
struct Vec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(p));
        f[0] = q.x, f[1] = q.y, f[2] = q.z, f[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    }
};

__device__ __forceinline__ float ld1(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ld1(const __half* p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void st1(float* p, float v) { *p = v; }
__device__ __forceinline__ void st1(__half* p, float v) { *p = __float2half_rn(v); }

// exp for the softmax numerator.  fp16 outputs carry 11 significant bits, so exp2f on a
// pre-scaled argument is ample there; fp32 outputs use expf.
template <typename T>
__device__ __forceinline__ float softmax_exp(float d);
template <>
__device__ __forceinline__ float softmax_exp<__half>(float d) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(d * 1.44269504088896340736f));
    return e;
}
template <>
__device__ __forceinline__ float softmax_exp<float>(float d) { return expf(d); }

// ---------------------------------------------------------------------------------------------
// Softmax: R rows per warp, the rows held in registers (ITERS packets per lane and row).  Short rows
// give a lane only a few 16-byte loads; taking several rows at once keeps enough bytes in flight per SM
// to cover the HBM latency, and interleaves the shuffle reductions of independent rows.
// ---------------------------------------------------------------------------------------------
template <typename T, int ITERS, int R>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ x, const T* __restrict__ mask,
                                                           T* __restrict__ y, int64_t rows, int cols,
                                                           int64_t mask_row_div, float scale, int is_log) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    constexpr int V = Vec<T>::N;
    const int lane = threadIdx.x & 31;
    const int64_t row0 = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
    if (row0 >= rows) return;
    float v[R][ITERS][V];
    float mx[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        mx[r] = -FLT_MAX;
        const int64_t row = row0 + r;
        if (row < rows) {
            const T* xr = x + row * cols;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int c = (it * 32 + lane) * V;
                if (c < cols) Vec<T>::load(xr + c, v[r][it]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int64_t row = row0 + r;
        if (row < rows) {
            const T* mr = mask ? mask + (row / mask_row_div) * cols : nullptr;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int c = (it * 32 + lane) * V;
                if (c < cols) {
                    if (mr) {
                        float mv[V];
                        Vec<T>::load(mr + c, mv);
#pragma unroll
                        for (int j = 0; j < V; ++j) v[r][it][j] = fmaf(v[r][it][j], scale, mv[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < V; ++j) v[r][it][j] *= scale;
                    }
#pragma unroll
                    for (int j = 0; j < V; ++j) mx[r] = fmaxf(mx[r], v[r][it][j]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) mx[r] = warp_max(mx[r]);
    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        sum[r] = 0.0f;
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int c = (it * 32 + lane) * V;
            if (c < cols) {
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const float d = v[r][it][j] - mx[r];
                    const float e = softmax_exp<T>(d);
                    sum[r] += e;
                    v[r][it][j] = is_log ? d : e;
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) sum[r] = warp_sum(sum[r]);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int64_t row = row0 + r;
        if (row < rows) {
            const float inv = 1.0f / sum[r];
            const float lse = logf(sum[r]);
            T* yr = y + row * cols;
#pragma unroll
            for (int it = 0; it < ITERS; ++it) {
                const int c = (it * 32 + lane) * V;
                if (c < cols) {
#pragma unroll
                    for (int j = 0; j < V; ++j) v[r][it][j] = is_log ? v[r][it][j] - lse : v[r][it][j] * inv;
                    Vec<T>::store(yr + c, v[r][it]);
                }
            }
        }
    }
}

// Any row length / alignment: one block per row, three passes over the row (it stays in L1/L2).
template <typename T>
__global__ void __launch_bounds__(256) softmax_block_kernel(const T* __restrict__ x, const T* __restrict__ mask,
                                                            T* __restrict__ y, int64_t cols, int64_t mask_row_div,
                                                            float scale, int is_log) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    __shared__ float red[8];
    __shared__ float bcast;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * cols;
    const T* mr = mask ? mask + (row / mask_row_div) * cols : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -FLT_MAX;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f);
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = red[0];
        for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
        bcast = m;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f);
        sum += softmax_exp<T>(v - mx);
    }
    sum = warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < 8; ++i) s += red[i];
        bcast = s;
    }
    __syncthreads();
    sum = bcast;
    const float inv = 1.0f / sum, lse = logf(sum);
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float d = ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f) - mx;
        st1(yr + c, is_log ? d - lse : softmax_exp<T>(d) * inv);
    }
}

// Short rows that the packet kernels cannot take (a length that is not a multiple of the packet, e.g. the 10 classes of
// a classifier head): LPR lanes share a row and a warp takes 32 / LPR rows, scalar loads served by the L1.  One block per
// row, the general fallback below, would launch thousands of nearly empty blocks for such a tensor.
template <typename T>
__global__ void __launch_bounds__(256) softmax_short_kernel(const T* __restrict__ x, const T* __restrict__ mask,
                                                            T* __restrict__ y, int64_t rows, int cols, int64_t mask_row_div,
                                                            float scale, int is_log, int lpr) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / lpr, l = lane - sub * lpr;
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * 8 + warp) * (32 / lpr) + sub;
    const bool valid = row < rows;  // lanes of rows past the end still take part in the shuffles
    const T* xr = x + (valid ? row : 0) * cols;
    const T* mr = mask ? mask + ((valid ? row : 0) / mask_row_div) * cols : nullptr;
    float mx = -FLT_MAX;
    for (int c = l; c < cols; c += lpr) mx = fmaxf(mx, ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f));
    for (int o = lpr >> 1; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (int c = l; c < cols; c += lpr) sum += softmax_exp<T>(ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f) - mx);
    for (int o = lpr >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (!valid) return;
    const float inv = 1.0f / sum, lse = logf(sum);
    T* yr = y + row * cols;
    for (int c = l; c < cols; c += lpr) {
        const float d = ld1(xr + c) * scale + (mr ? ld1(mr + c) : 0.0f) - mx;
        st1(yr + c, is_log ? d - lse : softmax_exp<T>(d) * inv);
    }
}

template <typename T>
int softmax_t(const T* x, const T* mask, T* y, int64_t rows, int64_t cols, int64_t mask_row_div, float scale,
              int is_log, cudaStream_t stream) {
    constexpr int V = Vec<T>::N;
    const bool vec = cols % V == 0 && aligned16(x) && aligned16(y) && (!mask || aligned16(mask));
    const int64_t packets = cols / V;
    if (vec && packets <= 32 * 8) {
        const int warps = 8;
        const int iters = (int)ceil_div(packets, 32);
        // two rows per warp while a row fits four packets per lane: more loads in flight, still 4-5 blocks per SM
        const int rpw = iters <= 4 ? 2 : 1;
        const int64_t blocks = ceil_div(rows, (int64_t)warps * rpw);
        B200ML_REQUIRE(blocks < (1ll << 31), "softmax: too many rows");
#define SM_LAUNCH(I, R)                                                                                          \
    launch_pdl(softmax_warp_kernel<T, I, R>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, x, mask, y, rows, (int)cols, mask_row_div, \
                                                                            scale, is_log)
        if (iters <= 1) SM_LAUNCH(1, 2);
        else if (iters <= 2) SM_LAUNCH(2, 2);
        else if (iters <= 4) SM_LAUNCH(4, 2);
        else SM_LAUNCH(8, 1);
#undef SM_LAUNCH
        return check_launch("softmax_warp");
    }
    if (cols <= 256) {
        int lpr = 4;
        while (lpr < 32 && lpr < cols) lpr <<= 1;
        const int64_t blocks = ceil_div(rows, (int64_t)8 * (32 / lpr));
        B200ML_REQUIRE(blocks < (1ll << 31), "softmax: too many rows");
        launch_pdl(softmax_short_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, x, mask, y, rows, (int)cols, mask_row_div, scale, is_log, lpr);
        return check_launch("softmax_short");
    }
    B200ML_REQUIRE(rows < (1ll << 31), "softmax: too many rows");
    launch_pdl(softmax_block_kernel<T>, dim3((unsigned)rows), dim3(256), 0, stream, x, mask, y, cols, mask_row_div, scale, is_log);
    return check_launch("softmax_block");
}

// ---------------------------------------------------------------------------------------------
// LayerNorm over the last axis of v = x (+ residual) (+ bias): mean, then the mean of squared
// deviations (two passes over registers, as the ReduceMean/Sub/Pow/ReduceMean chain does),
// eps added in fp32 (1e-12 underflows in fp16).
// ---------------------------------------------------------------------------------------------
template <typename T, int ITERS>
__global__ void __launch_bounds__(128) layernorm_warp_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                             const T* __restrict__ bias, const T* __restrict__ gamma,
                                                             const T* __restrict__ beta, T* __restrict__ y,
                                                             int64_t rows, int cols, float eps) {
    constexpr int V = Vec<T>::N;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* xr = x + row * cols;
    const T* rr = residual ? residual + row * cols : nullptr;
    float v[ITERS][V];
    float sum = 0.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * V;
        if (c < cols) {
            Vec<T>::load(xr + c, v[it]);
            if (rr) {
                float t[V];
                Vec<T>::load(rr + c, t);
#pragma unroll
                for (int j = 0; j < V; ++j) v[it][j] += t[j];
            }
            if (bias) {
                float t[V];
                Vec<T>::load(bias + c, t);
#pragma unroll
                for (int j = 0; j < V; ++j) v[it][j] += t[j];
            }
#pragma unroll
            for (int j = 0; j < V; ++j) sum += v[it][j];
        }
    }
    const float mean = warp_sum(sum) / cols;
    float sq = 0.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * V;
        if (c < cols) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                v[it][j] -= mean;
                sq = fmaf(v[it][j], v[it][j], sq);
            }
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / cols + eps);
    T* yr = y + row * cols;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
        const int c = (it * 32 + lane) * V;
        if (c < cols) {
            float gm[V], bt[V];
            if (gamma) Vec<T>::load(gamma + c, gm);
            if (beta) Vec<T>::load(beta + c, bt);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                float o = v[it][j] * rstd;
                if (gamma) o *= gm[j];
                if (beta) o += bt[j];
                v[it][j] = o;
            }
            Vec<T>::store(yr + c, v[it]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) layernorm_block_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                              const T* __restrict__ bias, const T* __restrict__ gamma,
                                                              const T* __restrict__ beta, T* __restrict__ y,
                                                              int64_t cols, float eps) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    __shared__ float red[8];
    __shared__ float bcast;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * cols;
    const T* rr = residual ? residual + row * cols : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto value = [&](int64_t c) { return ld1(xr + c) + (rr ? ld1(rr + c) : 0.0f) + (bias ? ld1(bias + c) : 0.0f); };
    float s = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += value(c);
    s = warp_sum(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; ++i) t += red[i];
        bcast = t / cols;
    }
    __syncthreads();
    const float mean = bcast;
    float sq = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float d = value(c) - mean;
        sq = fmaf(d, d, sq);
    }
    sq = warp_sum(sq);
    __syncthreads();
    if (lane == 0) red[warp] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int i = 0; i < 8; ++i) t += red[i];
        bcast = 1.0f / sqrtf(t / cols + eps);
    }
    __syncthreads();
    const float rstd = bcast;
    T* yr = y + row * cols;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        float o = (value(c) - mean) * rstd;
        if (gamma) o *= ld1(gamma + c);
        if (beta) o += ld1(beta + c);
        st1(yr + c, o);
    }
}

template <typename T>
int layernorm_t(const T* x, const T* residual, const T* bias, const T* gamma, const T* beta, T* y, int64_t rows,
                int64_t cols, float eps, cudaStream_t stream) {
    constexpr int V = Vec<T>::N;
    const bool vec = cols % V == 0 && aligned16(x) && aligned16(y) && (!residual || aligned16(residual)) &&
                     (!bias || aligned16(bias)) && (!gamma || aligned16(gamma)) && (!beta || aligned16(beta));
    const int64_t packets = cols / V;
    if (vec && packets <= 32 * 8) {
        const int warps = 4;
        const int64_t blocks = ceil_div(rows, warps);
        B200ML_REQUIRE(blocks < (1ll << 31), "layernorm: too many rows");
        const int iters = (int)ceil_div(packets, 32);
#define LN_LAUNCH(I)                                                                                             \
    B200ML_CUDA(launch_pdl(layernorm_warp_kernel<T, I>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream, x, residual, \
                           bias, gamma, beta, y, rows, (int)cols, eps))
        if (iters <= 1) LN_LAUNCH(1);
        else if (iters <= 2) LN_LAUNCH(2);
        else if (iters <= 4) LN_LAUNCH(4);
        else LN_LAUNCH(8);
#undef LN_LAUNCH
        return check_launch("layernorm_warp");
    }
    B200ML_REQUIRE(rows < (1ll << 31), "layernorm: too many rows");
    launch_pdl(layernorm_block_kernel<T>, dim3((unsigned)rows), dim3(256), 0, stream, x, residual, bias, gamma, beta, y, cols, eps);
    return check_launch("layernorm_block");
}

// ---------------------------------------------------------------------------------------------
// Reduce over the middle extent of [outer, reduce, inner]
// ---------------------------------------------------------------------------------------------
struct RedOp {
    int op;
    __device__ __forceinline__ float init() const {
        return op == B200ML_RED_MAX ? -FLT_MAX : (op == B200ML_RED_MIN ? FLT_MAX : 0.0f);
    }
    __device__ __forceinline__ float combine(float a, float b) const {
        return op == B200ML_RED_MAX ? fmaxf(a, b) : (op == B200ML_RED_MIN ? fminf(a, b) : a + b);
    }
    __device__ __forceinline__ float warp(float v) const {
        return op == B200ML_RED_MAX ? warp_max(v) : (op == B200ML_RED_MIN ? warp_min(v) : warp_sum(v));
    }
    __device__ __forceinline__ float finish(float v, int64_t n) const { return op == B200ML_RED_MEAN ? v / n : v; }
};

// inner == 1: contiguous rows.  One block per (row, slice); slices > 1 writes partials to scratch.
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                          float* __restrict__ partial, int64_t reduce, int slices,
                                                          RedOp op) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    __shared__ float red[8];
    const int64_t row = blockIdx.x;
    const int slice = blockIdx.y;
    const int64_t per = (reduce + slices - 1) / slices;
    const int64_t lo = slice * per, hi = lo + per < reduce ? lo + per : reduce;
    const T* xr = x + row * reduce;
    float v = op.init();
    for (int64_t c = lo + threadIdx.x; c < hi; c += blockDim.x) v = op.combine(v, ld1(xr + c));
    v = op.warp(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) t = op.combine(t, red[i]);
        if (slices == 1) st1(y + row, op.finish(t, reduce));
        else partial[row * slices + slice] = t;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) reduce_finish_kernel(const float* __restrict__ partial, T* __restrict__ y,
                                                            int64_t rows, int slices, int64_t reduce, RedOp op) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float v = op.init();
    for (int s = lane; s < slices; s += 32) v = op.combine(v, partial[row * slices + s]);
    v = op.warp(v);
    if (lane == 0) st1(y + row, op.finish(v, reduce));
}

// One warp per short contiguous row (GlobalAveragePool: rows of H*W).
template <typename T>
__global__ void __launch_bounds__(256) reduce_rows_warp_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                               int64_t rows, int64_t reduce, RedOp op) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * reduce;
    float v = op.init();
    constexpr int V = Vec<T>::N;
    if (reduce % V == 0 && (reinterpret_cast<uintptr_t>(xr) & 15u) == 0) {
        // 16-byte packets, four per lane in flight, each with its own partial result
        const int64_t packets = reduce / V;
        float acc[4] = {v, v, v, v};
        for (int64_t p = lane; p < packets; p += 128) {
            float f[4][V];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (p + 32 * u < packets) Vec<T>::load(xr + (p + 32 * u) * V, f[u]);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (p + 32 * u < packets) {
#pragma unroll
                    for (int j = 0; j < V; ++j) acc[u] = op.combine(acc[u], f[u][j]);
                }
            }
        }
        v = op.combine(op.combine(acc[0], acc[1]), op.combine(acc[2], acc[3]));
    } else {
        for (int64_t c = lane; c < reduce; c += 32) v = op.combine(v, ld1(xr + c));
    }
    v = op.warp(v);
    if (lane == 0) st1(y + row, op.finish(v, reduce));
}

// inner > 1: thread per (outer, inner) column, coalesced across inner.
template <typename T>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t outer,
                                                          int64_t reduce, int64_t inner, RedOp op) {
    pdl_launch_dependents();  // the next kernel of the stream may begin its set-up
    pdl_wait();               // everything before this kernel in the stream has completed
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= outer * inner) return;
    const int64_t o = idx / inner, i = idx % inner;
    const T* p = x + o * reduce * inner + i;
    float v = op.init();
    for (int64_t r = 0; r < reduce; ++r) v = op.combine(v, ld1(p + r * inner));
    st1(y + idx, op.finish(v, reduce));
}

template <typename T>
int reduce_t(const b200ml_ctx* ctx, int opcode, const T* x, T* y, int64_t outer, int64_t reduce, int64_t inner,
             cudaStream_t stream) {
    RedOp op{opcode};
    if (outer * inner == 0) return B200ML_OK;
    B200ML_REQUIRE(reduce > 0, "reduce: empty reduction extent");
    if (inner == 1) {
        if (reduce <= 4096) {
            const int64_t blocks = ceil_div(outer, 8);
            B200ML_REQUIRE(blocks < (1ll << 31), "reduce: too many rows");
            launch_pdl(reduce_rows_warp_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, x, y, outer, reduce, op);
            return check_launch("reduce_rows_warp");
        }
        // Long rows: cut each row into slices so that a full-tensor reduction still fills the GPU.
        int slices = 1;
        const int64_t want = 4ll * ctx->sm_count;
        if (outer < want) {
            slices = (int)((want + outer - 1) / outer);
            const int64_t max_by_len = reduce / 2048 > 0 ? reduce / 2048 : 1;
            if (slices > max_by_len) slices = (int)max_by_len;
            if (slices > 1024) slices = 1024;
        }
        B200ML_REQUIRE(outer < (1ll << 31), "reduce: too many rows");
        if (slices == 1) {
            launch_pdl(reduce_rows_kernel<T>, dim3(dim3((unsigned)outer, 1)), dim3(256), 0, stream, x, y, nullptr, reduce, 1, op);
            return check_launch("reduce_rows");
        }
        const int64_t need = outer * slices * (int64_t)sizeof(float);
        if (need > ctx->workspace_bytes)
            return fail(B200ML_ERR_WORKSPACE, "reduce: needs %lld bytes of scratch, the context has %lld",
                        (long long)need, (long long)ctx->workspace_bytes);
        float* partial = static_cast<float*>(ctx->workspace);
        launch_pdl(reduce_rows_kernel<T>, dim3(dim3((unsigned)outer, (unsigned)slices)), dim3(256), 0, stream, x, y, partial, reduce, slices, op);
        int rc = check_launch("reduce_rows");
        if (rc) return rc;
        launch_pdl(reduce_finish_kernel<T>, dim3((unsigned)ceil_div(outer, 8)), dim3(256), 0, stream, partial, y, outer, slices, reduce, op);
        return check_launch("reduce_finish");
    }
    const int64_t blocks = ceil_div(outer * inner, 256);
    B200ML_REQUIRE(blocks < (1ll << 31), "reduce: too many outputs");
    launch_pdl(reduce_cols_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, x, y, outer, reduce, inner, op);
    return check_launch("reduce_cols");
}

}  // namespace

int softmax(int dtype, const void* x, const void* mask, void* y, int64_t rows, int64_t cols, int64_t mask_row_div,
            float scale, int is_log, cudaStream_t s) {
    if (dtype == B200ML_F16)
        return softmax_t<__half>((const __half*)x, (const __half*)mask, (__half*)y, rows, cols, mask_row_div, scale, is_log, s);
    return softmax_t<float>((const float*)x, (const float*)mask, (float*)y, rows, cols, mask_row_div, scale, is_log, s);
}

int layernorm(int dtype, const void* x, const void* residual, const void* bias, const void* gamma, const void* beta,
              void* y, int64_t rows, int64_t cols, float eps, cudaStream_t s) {
    if (dtype == B200ML_F16)
        return layernorm_t<__half>((const __half*)x, (const __half*)residual, (const __half*)bias, (const __half*)gamma,
                                   (const __half*)beta, (__half*)y, rows, cols, eps, s);
    return layernorm_t<float>((const float*)x, (const float*)residual, (const float*)bias, (const float*)gamma,
                              (const float*)beta, (float*)y, rows, cols, eps, s);
}

int reduce(const b200ml_ctx* ctx, int dtype, int op, const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
           cudaStream_t s) {
    if (dtype == B200ML_F16) return reduce_t<__half>(ctx, op, (const __half*)x, (__half*)y, outer, red, inner, s);
    return reduce_t<float>(ctx, op, (const float*)x, (float*)y, outer, red, inner, s);
}

}  // namespace b200ml

// ---------------------------------------------------------------------------------------------
// Reduction that allocates nothing (b200ml_reduce_static)
// ---------------------------------------------------------------------------------------------
// The sliced long-row reduction needs a place for its per-slice partial results.  b200ml_reduce takes
// it from the context's scratch buffer, which b200ml_ctx_create obtained with cudaMalloc.  Some callers
// must not allocate device memory at all: code that runs while a CUDA graph is being captured or
// between the launches of a latency-critical serving loop (cudaMalloc synchronises the device and is
// illegal during capture), plug-ins that are handed a fixed memory budget by their host framework and
// may not grow it, and callers that run after the host allocator has been frozen.  For them the
// partials live in the array below, which is part of the library image: every GPU that loads the
// library holds these 4 KiB from load until the process exits.  1024 partial results cover every shape the
// slicing policy produces on a B200 except 513 to 591 long rows at once (two slices each).
constexpr int64_t kStaticScratchFloats = 1024;
static __device__ __align__(256) float g_reduce_static_scratch[kStaticScratchFloats];

namespace b200ml {
namespace {

constexpr int kMaxDevices = 64;
std::atomic<float*> g_static_scratch_ptr[kMaxDevices];
std::atomic<int> g_static_sm_count[kMaxDevices];

// In host code the array's name is only a handle for the runtime, not a device address; the address
// on the current device comes from cudaGetSymbolAddress.  Done once per device, on the first call
// made with that device current.
int static_scratch_for_current_device(float** ptr, int* sm_count) {
    int dev = 0;
    B200ML_CUDA(cudaGetDevice(&dev));
    B200ML_REQUIRE(dev >= 0 && dev < kMaxDevices, "reduce_static: device index %d out of range", dev);
    float* p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        void* sym = nullptr;
        B200ML_CUDA(cudaGetSymbolAddress(&sym, g_reduce_static_scratch));
        int sms = 0;
        B200ML_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_static_sm_count[dev].store(sms, std::memory_order_relaxed);
        p = static_cast<float*>(sym);
        g_static_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *ptr = p;
    *sm_count = g_static_sm_count[dev].load(std::memory_order_relaxed);
    return B200ML_OK;
}

}  // namespace
}  // namespace b200ml

extern "C" int b200ml_reduce_static(int32_t dtype, int32_t op, const void* x, void* y, int64_t outer, int64_t red,
                                    int64_t inner, b200ml_stream stream) {
    using namespace b200ml;
    B200ML_REQUIRE(dtype == B200ML_F16 || dtype == B200ML_F32, "reduce_static: unknown dtype %d", dtype);
    B200ML_REQUIRE(op >= B200ML_RED_SUM && op <= B200ML_RED_MIN, "reduce_static: unknown op %d", op);
    B200ML_REQUIRE(outer >= 0 && red >= 0 && inner >= 0, "reduce_static: negative extent");
    if (outer == 0 || inner == 0) return B200ML_OK;
    B200ML_REQUIRE(x && y, "reduce_static: null tensor");
    float* scratch = nullptr;
    int sms = 0;
    int rc = static_scratch_for_current_device(&scratch, &sms);
    if (rc) return rc;
    // A context that exists only on this stack frame: it points the shared reduction code at the static
    // array instead of an allocated buffer.  Nothing is allocated and nothing needs zeroing: the first
    // stage writes every partial the second stage reads.
    b200ml_ctx local;
    (void)cudaGetDevice(&local.device);
    local.sm_count = sms;
    local.workspace = scratch;
    local.workspace_bytes = kStaticScratchFloats * (int64_t)sizeof(float);
    rc = reduce(&local, dtype, op, x, y, outer, red, inner, static_cast<cudaStream_t>(stream));
    if (rc == B200ML_ERR_WORKSPACE)
        return fail(B200ML_ERR_WORKSPACE,
                    "reduce_static: %lld rows of %lld elements need more than the %lld partial sums of the built-in scratch "
                    "array; use b200ml_reduce with a context instead",
                    (long long)outer, (long long)red, (long long)kStaticScratchFloats);
    return rc;
}
