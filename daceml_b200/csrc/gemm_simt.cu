// FP32-FMA GEMM for the fp32 configurations (rtol 1e-4 rules out single-pass TF32) and for fp16
// operands whose layout the tensor-core kernel cannot address (unaligned leading dimensions,
// transposed A, tiny outputs).  Arbitrary row/column strides, two batch loops, same epilogue.
#include "common.cuh"
#include "epilogue.cuh"

namespace b200ml {

namespace {

constexpr int SBM = 64, SBN = 64, SBK = 16, STHREADS = 256;

template <typename T>
struct SimtArgs {
    int32_t m, n, k, batch_inner;
    int64_t a_rs, a_cs, a_so, a_si;  // A(m,k) = a[m*a_rs + k*a_cs]
    int64_t b_rs, b_cs, b_so, b_si;  // B(k,n) = b[k*b_rs + n*b_cs]
    int64_t ldc, c_so, c_si;
    int64_t ldr, r_so, r_si;
    EpilogueParams ep;
    const T* a;
    const T* b;
    const T* bias;
    const T* residual;
    T* c;
};

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__global__ void __launch_bounds__(STHREADS) gemm_simt_kernel(const SimtArgs<T> g) {
    __shared__ float As[SBK][SBM + 4];
    __shared__ float Bs[SBK][SBN + 4];
    const int tid = threadIdx.x;
    const int batch = blockIdx.z;
    const int bi = batch % g.batch_inner, bo = batch / g.batch_inner;
    const int m0 = blockIdx.y * SBM, n0 = blockIdx.x * SBN;
    const T* a = g.a + bo * g.a_so + bi * g.a_si;
    const T* b = g.b + bo * g.b_so + bi * g.b_si;

    // Thread-to-element maps for the tile loads: the contiguous axis of each operand goes to
    // consecutive threads.
    const bool a_k_contig = g.a_cs == 1;
    const bool b_n_contig = g.b_cs == 1;

    const int tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    // The next k-block's elements are fetched into registers while the current one is being multiplied: with one
    // 256-thread block per SM nothing else would cover the latency of the global loads.
    float ra[4], rb[4];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int mm, kk;
            if (a_k_contig) {
                kk = tid & 15;
                mm = (tid >> 4) + 16 * i;
            } else {
                mm = tid & 63;
                kk = (tid >> 6) + 4 * i;
            }
            const int gm = m0 + mm, gk = k0 + kk;
            ra[i] = (gm < g.m && gk < g.k) ? to_f(a[gm * g.a_rs + gk * g.a_cs]) : 0.0f;
            int nn, kb;
            if (b_n_contig) {
                nn = tid & 63;
                kb = (tid >> 6) + 4 * i;
            } else {
                kb = tid & 15;
                nn = (tid >> 4) + 16 * i;
            }
            const int gn = n0 + nn, gkb = k0 + kb;
            rb[i] = (gn < g.n && gkb < g.k) ? to_f(b[gkb * g.b_rs + gn * g.b_cs]) : 0.0f;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (a_k_contig) As[tid & 15][(tid >> 4) + 16 * i] = ra[i];
            else As[(tid >> 6) + 4 * i][tid & 63] = ra[i];
            if (b_n_contig) Bs[(tid >> 6) + 4 * i][tid & 63] = rb[i];
            else Bs[tid & 15][(tid >> 4) + 16 * i] = rb[i];
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < g.k; k0 += SBK) {
        stash();
        __syncthreads();
        if (k0 + SBK < g.k) fetch(k0 + SBK);
#pragma unroll
        for (int kk = 0; kk < SBK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float aa[4] = {av.x, av.y, av.z, av.w};
            const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(aa[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }

    T* c = g.c + bo * g.c_so + bi * g.c_si;
    const T* res = g.residual ? g.residual + bo * g.r_so + bi * g.r_si : nullptr;
    const bool has_bias = (g.ep.flags & B200ML_EPI_BIAS) && g.bias;
    const bool has_res = (g.ep.flags & B200ML_EPI_RESIDUAL) && res;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= g.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= g.n) continue;
            float v = g.ep.alpha * acc[i][j];
            if (has_bias) v = fmaf(g.ep.bias_scale, to_f(g.bias[gn]), v);
            v = apply_act(v, g.ep.flags);
            if (has_res) v = fmaf(g.ep.residual_scale, to_f(res[gm * g.ldr + gn]), v);
            c[gm * g.ldc + gn] = from_f<T>(v);
        }
    }
}

template <typename T>
int launch_simt(const b200ml_gemm_params* p, cudaStream_t stream) {
    SimtArgs<T> g{};
    g.m = (int32_t)p->m;
    g.n = (int32_t)p->n;
    g.k = (int32_t)p->k;
    g.batch_inner = (int32_t)p->batch_inner;
    if (p->a_layout == 0) {
        g.a_rs = p->lda;
        g.a_cs = 1;
    } else {
        g.a_rs = 1;
        g.a_cs = p->lda;
    }
    if (p->b_layout == 0) {
        g.b_rs = p->ldb;
        g.b_cs = 1;
    } else {
        g.b_rs = 1;
        g.b_cs = p->ldb;
    }
    g.a_so = p->a_stride_outer;
    g.a_si = p->a_stride_inner;
    g.b_so = p->b_stride_outer;
    g.b_si = p->b_stride_inner;
    g.ldc = p->ldc;
    g.c_so = p->c_stride_outer;
    g.c_si = p->c_stride_inner;
    g.ldr = p->ldr;
    g.r_so = p->r_stride_outer;
    g.r_si = p->r_stride_inner;
    g.ep.flags = p->epilogue;
    g.ep.alpha = p->alpha;
    g.ep.bias_scale = p->bias_scale;
    g.ep.residual_scale = p->residual_scale;
    g.a = static_cast<const T*>(p->a);
    g.b = static_cast<const T*>(p->b);
    g.bias = static_cast<const T*>(p->bias);
    g.residual = static_cast<const T*>(p->residual);
    g.c = static_cast<T*>(p->c);
    const int64_t batches = p->batch_outer * p->batch_inner;
    B200ML_REQUIRE(batches <= 65535 && ceil_div(p->m, SBM) <= 65535, "gemm: grid too large for the FP32-FMA kernel");
    dim3 grid((unsigned)ceil_div(p->n, SBN), (unsigned)ceil_div(p->m, SBM), (unsigned)batches);
    gemm_simt_kernel<T><<<grid, STHREADS, 0, stream>>>(g);
    return check_launch("gemm_simt");
}

// ---------------------------------------------------------------------------------------------
// Skinny outputs (N <= 16: classifier heads, the last layer of an MLP): the 64 x 64 tile above leaves most of its columns
// empty.  (At N = 32 this kernel was measured no faster than the tile kernel - 13.5 vs 11.1 us for 4096 x 32 x 120 - so
// the tile kernel keeps those.)  Here the whole B matrix sits in shared memory as Ws[k][NP], a
// thread owns one row of A and eight output columns, and A is read once with 16-byte loads.
// ---------------------------------------------------------------------------------------------
struct SkinnyArgs {
    int32_t m, n, k, np;   // np = n rounded up to a multiple of 8
    int32_t ws_stride;     // floats between consecutive k rows of the copy of B (np + 4: transposed fills spread over banks)
    int64_t lda, b_rs, b_cs, ldc, ldr;
    EpilogueParams ep;
    const float* a;
    const float* b;
    const float* bias;
    const float* residual;
    float* c;
};

__global__ void __launch_bounds__(256) gemm_skinny_f32_kernel(const SkinnyArgs g) {
    extern __shared__ __align__(16) float ws[];  // [k][ws_stride]
    if (g.b_cs == 1) {  // B is [K, N]: consecutive threads walk a row of it
        for (int i = threadIdx.x; i < g.k * g.np; i += blockDim.x) {
            const int kk = i / g.np, nn = i - kk * g.np;
            ws[kk * g.ws_stride + nn] = nn < g.n ? __ldg(g.b + kk * g.b_rs + nn) : 0.0f;
        }
    } else {  // B is [N, K] (nn.Linear weights): consecutive threads walk k, the contiguous axis
        for (int i = threadIdx.x; i < g.k * g.np; i += blockDim.x) {
            const int nn = i / g.k, kk = i - nn * g.k;
            ws[kk * g.ws_stride + nn] = nn < g.n ? __ldg(g.b + nn * g.b_cs + kk) : 0.0f;
        }
    }
    __syncthreads();
    const int tpr = g.np >> 3;  // threads per row
    const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x / tpr) + threadIdx.x / tpr;
    const int n0 = (threadIdx.x % tpr) * 8;
    if (row >= g.m || threadIdx.x / tpr >= blockDim.x / tpr) return;
    const float4* ar = reinterpret_cast<const float4*>(g.a + row * g.lda);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 4  // four independent 16-byte loads of A in flight: there are only a few warps per SM to hide them
    for (int k4 = 0; k4 < g.k / 4; ++k4) {
        const float4 av = __ldg(ar + k4);
        const float aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float4* wr = reinterpret_cast<const float4*>(ws + (k4 * 4 + t) * g.ws_stride + n0);
            const float4 w0 = wr[0], w1 = wr[1];
            acc[0] = fmaf(aa[t], w0.x, acc[0]), acc[1] = fmaf(aa[t], w0.y, acc[1]);
            acc[2] = fmaf(aa[t], w0.z, acc[2]), acc[3] = fmaf(aa[t], w0.w, acc[3]);
            acc[4] = fmaf(aa[t], w1.x, acc[4]), acc[5] = fmaf(aa[t], w1.y, acc[5]);
            acc[6] = fmaf(aa[t], w1.z, acc[6]), acc[7] = fmaf(aa[t], w1.w, acc[7]);
        }
    }
    const bool has_bias = (g.ep.flags & B200ML_EPI_BIAS) && g.bias;
    const bool has_res = (g.ep.flags & B200ML_EPI_RESIDUAL) && g.residual;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int gn = n0 + j;
        if (gn >= g.n) break;
        float v = g.ep.alpha * acc[j];
        if (has_bias) v = fmaf(g.ep.bias_scale, __ldg(g.bias + gn), v);
        v = apply_act(v, g.ep.flags);
        if (has_res) v = fmaf(g.ep.residual_scale, __ldg(g.residual + row * g.ldr + gn), v);
        g.c[row * g.ldc + gn] = v;
    }
}

bool skinny_applies(const b200ml_gemm_params* p) {
    return p->dtype == B200ML_F32 && p->batch_outer * p->batch_inner == 1 && p->a_layout == 0 && p->n <= 16 && p->k % 4 == 0 &&
           p->lda % 4 == 0 && aligned16(p->a) && p->k * ((p->n + 7) / 8 * 8 + 4) * 4 <= 48 * 1024 && p->m >= 256 &&
           !(p->epilogue & B200ML_EPI_LAYERNORM);
}

int launch_skinny(const b200ml_gemm_params* p, cudaStream_t stream) {
    SkinnyArgs g{};
    g.m = (int32_t)p->m, g.n = (int32_t)p->n, g.k = (int32_t)p->k, g.np = (int32_t)((p->n + 7) / 8 * 8);
    g.ws_stride = g.np + 4;
    g.lda = p->lda, g.ldc = p->ldc, g.ldr = p->ldr;
    g.b_rs = p->b_layout == 0 ? p->ldb : 1;  // B(k, n) = b[k * b_rs + n * b_cs]
    g.b_cs = p->b_layout == 0 ? 1 : p->ldb;
    g.ep.flags = p->epilogue, g.ep.alpha = p->alpha, g.ep.bias_scale = p->bias_scale, g.ep.residual_scale = p->residual_scale;
    g.a = static_cast<const float*>(p->a), g.b = static_cast<const float*>(p->b);
    g.bias = static_cast<const float*>(p->bias), g.residual = static_cast<const float*>(p->residual);
    g.c = static_cast<float*>(p->c);
    const int tpr = g.np / 8;
    // 128 threads per block: the copy of B into shared memory is per block, but so is the latency of its first loads
    const int threads = 128;
    const int rows_per_block = threads / tpr;
    const size_t smem = static_cast<size_t>(g.k) * g.ws_stride * sizeof(float);
    gemm_skinny_f32_kernel<<<(unsigned)ceil_div(p->m, rows_per_block), threads, smem, stream>>>(g);
    return check_launch("gemm_skinny");
}

}  // namespace

bool gemm_f32_tensor_core_applies(const b200ml_ctx* ctx, const b200ml_gemm_params* p);
int gemm_f32_tensor_core(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream);

// Large K-major fp32 products run on the tensor cores as three TF32 passes (fp32-grade accuracy); the rest here.
int gemm_f32(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream) {
    if (gemm_f32_tensor_core_applies(ctx, p)) return gemm_f32_tensor_core(ctx, p, stream);
    if (skinny_applies(p)) return launch_skinny(p, stream);
    return launch_simt<float>(p, stream);
}
int gemm_f16_simt(const b200ml_ctx*, const b200ml_gemm_params* p, cudaStream_t stream) {
    return launch_simt<__half>(p, stream);
}

}  // namespace b200ml
