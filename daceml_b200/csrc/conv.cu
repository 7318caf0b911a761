// ONNX Conv (NCHW cross-correlation) and squeeze-excite, FP32 FMA (rtol 1e-4 rules out TF32).
//   * pointwise_x / pointwise_acc: 1x1 stride-1 convolutions as per-pixel small matrix products,
//     four pixels per thread, weights broadcast from shared memory, one read of X and one write
//     of Y; bias, Swish/ReLU, squeeze-excite gate on the input and the residual add are fused.
//   * depthwise_plane: one (image, channel) plane per block staged in shared memory with its
//     halo; bias + activation and the GlobalAveragePool of the result are fused.
//   * direct: any stride / pad / dilation / group; accumulates in (c, i, j) order like the
//     reference's 7-deep loop nest (daceml/onnx/op_implementations/img_op_implementations.py:263-288).
#include "common.cuh"
#include "epilogue.cuh"

namespace b200ml {

int reduce(const b200ml_ctx* ctx, int dtype, int op, const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
           cudaStream_t s);
bool conv1x1_tensor_core_applies(const b200ml_ctx* ctx, const b200ml_conv_params* p);
int conv1x1_tensor_core(const b200ml_ctx* ctx, const b200ml_conv_params* p, cudaStream_t stream);
bool conv_igemm_applies(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t oh, int64_t ow);
int conv_igemm(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t oh, int64_t ow, cudaStream_t stream);
int64_t conv1x1_pack_bytes(const b200ml_conv_params* p);
int conv1x1_pack(const b200ml_ctx* ctx, const b200ml_conv_params* p, void* dst, cudaStream_t stream);
int64_t conv_igemm_pack_bytes(const b200ml_conv_params* p, int64_t ow);
int conv_igemm_pack(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t ow, void* dst, cudaStream_t stream);

namespace {

__device__ __forceinline__ float ldv(const float* p) { return __ldg(p); }
__device__ __forceinline__ float ldv(const __half* p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ void stv(float* p, float v) { *p = v; }
__device__ __forceinline__ void stv(__half* p, float v) { *p = __float2half_rn(v); }

struct ConvGeom {
    int32_t n, c, h, w, m, kh, kw, sh, sw, pt, pl, dh, dw, group, oh, ow, act;
};

// ---------------------------------------------------------------------------------------------
// direct convolution: one thread = one output pixel x MT consecutive output channels
// ---------------------------------------------------------------------------------------------
constexpr int MT = 8;

// K = 3: 3x3 taps known at compile time, so the nine loads of a channel are issued together instead of one
// dependent L2 round trip per tap; K = 0: any kernel size.  The MT x (C/group) x kh x kw weights of the block's
// output channels are staged in shared memory when they fit (WSM floats).
constexpr int WSM = 2048;

template <typename T, int K>
__global__ void __launch_bounds__(256) conv_direct_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                          const T* __restrict__ bias, const T* __restrict__ gate,
                                                          const T* __restrict__ residual, T* __restrict__ y,
                                                          const ConvGeom g) {
    __shared__ float wsm[WSM];
    const int cg = g.c / g.group;   // input channels per group
    const int mg = g.m / g.group;   // output channels per group
    const int mblocks = (mg + MT - 1) / MT;
    const int grp = blockIdx.y / mblocks;
    const int m0 = grp * mg + (blockIdx.y % mblocks) * MT;
    const int mend = (grp + 1) * mg;
    const int kh = K ? K : g.kh, kw = K ? K : g.kw;
    const int wstride = cg * kh * kw;  // weights per output channel
    const bool w_in_smem = MT * wstride <= WSM;
    if (w_in_smem) {
        for (int i = threadIdx.x; i < MT * wstride; i += blockDim.x) {
            const int t = i / wstride;
            wsm[i] = m0 + t < mend ? ldv(w + static_cast<int64_t>(m0 + t) * wstride + (i - t * wstride)) : 0.0f;
        }
        __syncthreads();
    }
    const int64_t pix = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t npix = static_cast<int64_t>(g.n) * g.oh * g.ow;
    if (pix >= npix) return;
    const int ox = pix % g.ow;
    const int oy = (pix / g.ow) % g.oh;
    const int b = pix / (static_cast<int64_t>(g.ow) * g.oh);
    float acc[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) acc[t] = (bias && m0 + t < mend) ? ldv(bias + m0 + t) : 0.0f;
    for (int c = 0; c < cg; ++c) {
        const int ci = grp * cg + c;
        const T* xp = x + (static_cast<int64_t>(b) * g.c + ci) * g.h * g.w;
        const float gt = gate ? ldv(gate + static_cast<int64_t>(b) * g.c + ci) : 1.0f;
        if (K == 3) {
            float xv[9];
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int iy = oy * g.sh - g.pt + i * g.dh;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int ix = ox * g.sw - g.pl + j * g.dw;
                    const bool in = iy >= 0 && iy < g.h && ix >= 0 && ix < g.w;
                    xv[i * 3 + j] = in ? ldv(xp + static_cast<int64_t>(iy) * g.w + ix) * gt : 0.0f;
                }
            }
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    const float wv = w_in_smem ? wsm[t * wstride + c * 9 + tap]
                                               : (m0 + t < mend ? ldv(w + static_cast<int64_t>(m0 + t) * wstride + c * 9 + tap) : 0.0f);
                    acc[t] = fmaf(wv, xv[tap], acc[t]);
                }
            }
        } else {
            for (int i = 0; i < kh; ++i) {
                const int iy = oy * g.sh - g.pt + i * g.dh;
                if (iy < 0 || iy >= g.h) continue;
                for (int j = 0; j < kw; ++j) {
                    const int ix = ox * g.sw - g.pl + j * g.dw;
                    if (ix < 0 || ix >= g.w) continue;
                    const float xv = ldv(xp + static_cast<int64_t>(iy) * g.w + ix) * gt;
                    const int wo = (c * kh + i) * kw + j;
#pragma unroll
                    for (int t = 0; t < MT; ++t) {
                        const float wv = w_in_smem ? wsm[t * wstride + wo]
                                                   : (m0 + t < mend ? ldv(w + static_cast<int64_t>(m0 + t) * wstride + wo) : 0.0f);
                        acc[t] = fmaf(wv, xv, acc[t]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        if (m0 + t < mend) {
            const int64_t o = ((static_cast<int64_t>(b) * g.m + m0 + t) * g.oh + oy) * g.ow + ox;
            float v = conv_act(acc[t], g.act);
            if (residual) v += ldv(residual + o);
            stv(y + o, v);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// 1x1 convolution, few input channels (C <= 32): X held in registers, loop over output channels
// ---------------------------------------------------------------------------------------------
template <int CP>  // C padded to a multiple of 4
__global__ void __launch_bounds__(128) pointwise_x_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                          const float* __restrict__ bias, const float* __restrict__ gate,
                                                          const float* __restrict__ residual, float* __restrict__ y,
                                                          int64_t total4, int p4, int c, int m, int act) {
    extern __shared__ float wsm[];  // [m_part][CP], zero-padded: this block's share of the output channels
    const int m_part = (m + gridDim.y - 1) / gridDim.y;
    const int m_begin = blockIdx.y * m_part;
    const int m_end = m_begin + m_part < m ? m_begin + m_part : m;
    for (int i = threadIdx.x; i < (m_end - m_begin) * CP; i += blockDim.x) {
        const int mm = i / CP, cc = i % CP;
        wsm[i] = cc < c ? __ldg(w + (m_begin + mm) * c + cc) : 0.0f;
    }
    __syncthreads();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int64_t img = idx / p4;
    const int q = idx % p4;
    const float4* xp = reinterpret_cast<const float4*>(x) + img * c * p4 + q;
    float4 xv[CP];
#pragma unroll
    for (int cc = 0; cc < CP; ++cc) {
        if (cc < c) {
            xv[cc] = __ldg(xp + static_cast<int64_t>(cc) * p4);
            if (gate) {
                const float gt = __ldg(gate + img * c + cc);
                xv[cc].x *= gt, xv[cc].y *= gt, xv[cc].z *= gt, xv[cc].w *= gt;
            }
        } else {
            xv[cc] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float4* yp = reinterpret_cast<float4*>(y) + img * m * p4 + q;
    const float4* rp = residual ? reinterpret_cast<const float4*>(residual) + img * m * p4 + q : nullptr;
    for (int mm = m_begin; mm < m_end; ++mm) {
        const float b = bias ? __ldg(bias + mm) : 0.0f;
        float4 acc = make_float4(b, b, b, b);
        const float4* wr = reinterpret_cast<const float4*>(wsm + (mm - m_begin) * CP);
#pragma unroll
        for (int c4 = 0; c4 < CP / 4; ++c4) {
            const float4 wv = wr[c4];
            const float ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float4 xx = xv[c4 * 4 + t];
                acc.x = fmaf(ws[t], xx.x, acc.x);
                acc.y = fmaf(ws[t], xx.y, acc.y);
                acc.z = fmaf(ws[t], xx.z, acc.z);
                acc.w = fmaf(ws[t], xx.w, acc.w);
            }
        }
        acc.x = conv_act(acc.x, act), acc.y = conv_act(acc.y, act);
        acc.z = conv_act(acc.z, act), acc.w = conv_act(acc.w, act);
        if (rp) {
            const float4 r = __ldg(rp + static_cast<int64_t>(mm) * p4);
            acc.x += r.x, acc.y += r.y, acc.z += r.z, acc.w += r.w;
        }
        yp[static_cast<int64_t>(mm) * p4] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// 1x1 convolution, few output channels per pass (MP <= 32): accumulators in registers, loop over C
// ---------------------------------------------------------------------------------------------
constexpr int ACC_CH = 4;      // input channels per ring stage
constexpr int ACC_STAGES = 4;  // ring depth: 3 x 4 loads of 16 bytes in flight per thread
constexpr size_t ACC_SMEM_LIMIT = 96 * 1024;  // weights of one pass (c x MP floats) + the rings
constexpr size_t ACC_RING_BYTES = static_cast<size_t>(ACC_STAGES) * ACC_CH * 128 * sizeof(float4);

template <int MP>  // output channels per pass, multiple of 4
__global__ void __launch_bounds__(128) pointwise_acc_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            const float* __restrict__ bias,
                                                            const float* __restrict__ gate,
                                                            const float* __restrict__ residual, float* __restrict__ y,
                                                            int64_t total4, int p4, int c, int m, int act) {
    extern __shared__ float wsm[];  // [c][MP]: the MP weights of one input channel are contiguous
    const int m0 = blockIdx.y * MP;
    for (int i = threadIdx.x; i < c * MP; i += blockDim.x) {
        const int cc = i / MP, mm = i % MP;
        wsm[i] = (m0 + mm < m) ? __ldg(w + static_cast<int64_t>(m0 + mm) * c + cc) : 0.0f;
    }
    __syncthreads();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int64_t img = idx / p4;
    const int q = idx % p4;
    const float4* xp = reinterpret_cast<const float4*>(x) + img * c * p4 + q;
    const float* gp = gate ? gate + img * c : nullptr;
    float4 acc[MP];
#pragma unroll
    for (int mm = 0; mm < MP; ++mm) {
        const float b = (bias && m0 + mm < m) ? __ldg(bias + m0 + mm) : 0.0f;
        acc[mm] = make_float4(b, b, b, b);
    }
    // The accumulators take the registers, so the loads of X run ahead through shared memory instead: every thread owns
    // a ring of ACC_STAGES x ACC_CH 16-byte slots that it fills with cp.async and reads back itself (no barrier), which
    // keeps (ACC_STAGES - 1) * ACC_CH loads per thread in flight whatever the occupancy.
    float4* ring = reinterpret_cast<float4*>(wsm + ((c * MP + 3) & ~3)) + threadIdx.x;
    auto issue = [&](int chunk) {
        const int slot = (chunk % ACC_STAGES) * ACC_CH;
#pragma unroll
        for (int k = 0; k < ACC_CH; ++k) {
            const int cc = chunk * ACC_CH + k;
            if (cc < c) {
                const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(ring + (slot + k) * 128));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(xp + static_cast<int64_t>(cc) * p4) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int chunks = (c + ACC_CH - 1) / ACC_CH;
#pragma unroll
    for (int pre = 0; pre < ACC_STAGES - 1; ++pre) issue(pre);  // chunks beyond the end commit empty groups
    for (int chunk = 0; chunk < chunks; ++chunk) {
        issue(chunk + ACC_STAGES - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(ACC_STAGES - 1) : "memory");
        const int slot = (chunk % ACC_STAGES) * ACC_CH;
#pragma unroll
        for (int k = 0; k < ACC_CH; ++k) {
            const int cc = chunk * ACC_CH + k;
            if (cc >= c) break;
            float4 xx = ring[(slot + k) * 128];
            if (gp) {
                const float gt = __ldg(gp + cc);
                xx.x *= gt, xx.y *= gt, xx.z *= gt, xx.w *= gt;
            }
            const float4* wr = reinterpret_cast<const float4*>(wsm + cc * MP);
#pragma unroll
            for (int m4 = 0; m4 < MP / 4; ++m4) {
                const float4 wv = wr[m4];
                const float ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    float4& a = acc[m4 * 4 + t];
                    a.x = fmaf(ws[t], xx.x, a.x);
                    a.y = fmaf(ws[t], xx.y, a.y);
                    a.z = fmaf(ws[t], xx.z, a.z);
                    a.w = fmaf(ws[t], xx.w, a.w);
                }
            }
        }
    }
    float4* yp = reinterpret_cast<float4*>(y) + img * m * p4 + q;
    const float4* rp = residual ? reinterpret_cast<const float4*>(residual) + img * m * p4 + q : nullptr;
#pragma unroll
    for (int mm = 0; mm < MP; ++mm) {
        if (m0 + mm < m) {
            float4 a = acc[mm];
            if (act) a.x = conv_act(a.x, act), a.y = conv_act(a.y, act), a.z = conv_act(a.z, act), a.w = conv_act(a.w, act);
            if (rp) {
                const float4 r = __ldg(rp + static_cast<int64_t>(m0 + mm) * p4);
                a.x += r.x, a.y += r.y, a.z += r.z, a.w += r.w;
            }
            yp[static_cast<int64_t>(m0 + mm) * p4] = a;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// depthwise convolution, stride 1: one (image, channel) plane per block
// ---------------------------------------------------------------------------------------------
// 3x3, unit stride and dilation, planes up to 64 pixels wide: no shared memory.  A lane owns one output column of a
// strip of rows and slides a 3x3 window down it - three (L1-served) loads, nine multiply-adds, one store per output,
// against the 130 instructions per output of the staged kernel below (index arithmetic and shared-memory traffic).
__global__ void __launch_bounds__(256) depthwise3x3_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           const float* __restrict__ bias, float* __restrict__ y,
                                                           float* __restrict__ pool_mean, const ConvGeom g) {
    __shared__ float red[8];
    const int ch = blockIdx.x % g.c;
    const int64_t img = blockIdx.x / g.c;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* xp = x + (img * g.c + ch) * static_cast<int64_t>(g.h) * g.w;
    float* yp = y + (img * g.m + ch) * static_cast<int64_t>(g.oh) * g.ow;
    float t[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) t[i] = __ldg(w + ch * 9 + i);
    const float b = bias ? __ldg(bias + ch) : 0.0f;
    const int ox = lane + 32 * (warp & 1);
    const bool col_ok = ox < g.ow;
    const int rows_per = (g.oh + 3) >> 2;  // four strips of rows
    const int oy0 = (warp >> 1) * rows_per;
    const int oy1 = oy0 + rows_per < g.oh ? oy0 + rows_per : g.oh;
    const int ix0 = ox - g.pl;
    auto load_row = [&](int iy, float (&v)[3]) {
        const bool row_in = col_ok && iy >= 0 && iy < g.h;
        const float* rp = xp + static_cast<int64_t>(iy) * g.w;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int ix = ix0 + j;
            v[j] = (row_in && ix >= 0 && ix < g.w) ? __ldg(rp + ix) : 0.0f;
        }
    };
    // four output rows per step: the twelve loads of the next four input rows are issued before the first
    // multiply, so that each thread keeps enough bytes in flight to cover the HBM latency
    float r[6][3];
    load_row(oy0 - g.pt, r[0]);
    load_row(oy0 - g.pt + 1, r[1]);
    float local = 0.0f;
    for (int oy = oy0; oy < oy1; oy += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) load_row(oy + k - g.pt + 2, r[2 + k]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float acc = b;
#pragma unroll
            for (int i = 0; i < 3; ++i)
#pragma unroll
                for (int j = 0; j < 3; ++j) acc = fmaf(t[i * 3 + j], r[k + i][j], acc);
            acc = conv_act(acc, g.act);
            if (col_ok && oy + k < oy1) {
                yp[(oy + k) * g.ow + ox] = acc;
                local += acc;
            }
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) r[0][j] = r[4][j], r[1][j] = r[5][j];
    }
    if (pool_mean) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0) red[warp] = local;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int i = 0; i < 8; ++i) tot += red[i];
            pool_mean[img * g.m + ch] = tot / (g.oh * g.ow);
        }
    }
}

// 3x3, unit stride, pad 1 on every side, width a multiple of 4 up to 64: a lane owns FOUR adjacent output columns of a
// strip of rows.  Per input row it issues one 16-byte load; the two halo columns come from the neighbouring lanes by
// shuffle (zero at the plane's edges), so four outputs cost one load, two shuffles, 36 multiply-adds and one 16-byte
// store - a quarter of the instructions of the column-per-lane kernel above, which is bound by instruction issue.
// One warp per plane: LPR = w / 4 lanes cover a row, 32 / LPR strips of rows share the warp.
__global__ void __launch_bounds__(128) depthwise3x3_quad_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                const float* __restrict__ bias, float* __restrict__ y,
                                                                float* __restrict__ pool_mean, const ConvGeom g,
                                                                int64_t planes) {
    const int lane = threadIdx.x & 31;
    const int64_t plane = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (plane >= planes) return;  // whole warps leave; no block-wide barrier below
    const int ch = static_cast<int>(plane % g.c);
    const int64_t img = plane / g.c;
    const int lpr = g.w >> 2;            // lanes per row
    const int strips = 32 / lpr;         // row strips per warp
    const int strip = lane / lpr, q = lane - strip * lpr;
    const bool active = strip < strips;
    const int rows_per = (g.h + strips - 1) / strips;
    const int oy0 = strip * rows_per;
    const int oy1 = active ? (oy0 + rows_per < g.h ? oy0 + rows_per : g.h) : oy0;
    const float4* xp = reinterpret_cast<const float4*>(x + (img * g.c + ch) * static_cast<int64_t>(g.h) * g.w) + q;
    float4* yp = reinterpret_cast<float4*>(y + (img * g.m + ch) * static_cast<int64_t>(g.h) * g.w) + q;
    float t[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) t[i] = __ldg(w + ch * 9 + i);
    const float b = bias ? __ldg(bias + ch) : 0.0f;

    // a row as this lane sees it: left halo, four own columns, right halo
    struct Row { float v[6]; };
    auto fetch = [&](int iy) -> float4 {
        return (active && iy >= 0 && iy < g.h) ? __ldg(xp + static_cast<int64_t>(iy) * lpr) : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    auto finish = [&](const float4& c) -> Row {
        Row r;
        // every lane takes part in the shuffles (inactive lanes hold zeros); edges of the plane read the padding
        const float left = __shfl_up_sync(0xffffffffu, c.w, 1);
        const float right = __shfl_down_sync(0xffffffffu, c.x, 1);
        r.v[0] = q == 0 ? 0.0f : left;
        r.v[1] = c.x, r.v[2] = c.y, r.v[3] = c.z, r.v[4] = c.w;
        r.v[5] = q == lpr - 1 ? 0.0f : right;
        return r;
    };
    auto output = [&](const Row& r0, const Row& r1, const Row& r2) -> float4 {
        float o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float acc = b;
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                acc = fmaf(t[j], r0.v[k + j], acc);
                acc = fmaf(t[3 + j], r1.v[k + j], acc);
                acc = fmaf(t[6 + j], r2.v[k + j], acc);
            }
            o[k] = conv_act(acc, g.act);
        }
        return make_float4(o[0], o[1], o[2], o[3]);
    };

    // the strips of a warp have the same number of steps (rows_per), so the shuffles stay warp-uniform
    Row ra = finish(fetch(oy0 - 1)), rb = finish(fetch(oy0));
    float local = 0.0f;
    for (int k = 0; k < rows_per; k += 2) {
        const int oy = oy0 + k;
        const float4 c0 = fetch(oy + 1), c1 = fetch(oy + 2);  // both loads in flight before the first multiply
        const Row rc = finish(c0), rd = finish(c1);
        if (oy < oy1) {
            const float4 o = output(ra, rb, rc);
            yp[static_cast<int64_t>(oy) * lpr] = o;
            local += (o.x + o.y) + (o.z + o.w);
        }
        if (oy + 1 < oy1) {
            const float4 o = output(rb, rc, rd);
            yp[static_cast<int64_t>(oy + 1) * lpr] = o;
            local += (o.x + o.y) + (o.z + o.w);
        }
        ra = rc, rb = rd;
    }
    if (pool_mean) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0) pool_mean[img * g.m + ch] = local / (g.h * g.w);
    }
}

// Any kernel size up to 64 taps: the plane and its halo staged in shared memory.  Warps walk rows and lanes walk
// columns, so no index needs a division.
__global__ void __launch_bounds__(256) depthwise_plane_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                              const float* __restrict__ bias, float* __restrict__ y,
                                                              float* __restrict__ pool_mean, const ConvGeom g) {
    extern __shared__ float plane[];  // (h + kh - 1 ... ) padded input plane
    __shared__ float red[8];
    __shared__ float wk[64];
    const int ch = blockIdx.x % g.c;
    const int64_t img = blockIdx.x / g.c;
    const int kh = g.kh, kw = g.kw;
    const int ph = g.oh + kh - 1, pw = g.ow + kw - 1;  // padded plane extents actually read
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* xp = x + (img * g.c + ch) * static_cast<int64_t>(g.h) * g.w;
    for (int py = warp; py < ph; py += 8) {
        const int iy = py - g.pt;
        const bool row_in = iy >= 0 && iy < g.h;
        for (int px = lane; px < pw; px += 32) {
            const int ix = px - g.pl;
            plane[py * pw + px] = (row_in && ix >= 0 && ix < g.w) ? __ldg(xp + iy * g.w + ix) : 0.0f;
        }
    }
    if (threadIdx.x < kh * kw) wk[threadIdx.x] = __ldg(w + ch * kh * kw + threadIdx.x);
    __syncthreads();
    const float b = bias ? __ldg(bias + ch) : 0.0f;
    float* yp = y + (img * g.m + ch) * static_cast<int64_t>(g.oh) * g.ow;
    float local = 0.0f;
    for (int oy = warp; oy < g.oh; oy += 8) {
        for (int ox = lane; ox < g.ow; ox += 32) {
            float acc = b;
            for (int i = 0; i < kh; ++i)
                for (int j = 0; j < kw; ++j) acc = fmaf(wk[i * kw + j], plane[(oy + i) * pw + ox + j], acc);
            acc = conv_act(acc, g.act);
            yp[oy * g.ow + ox] = acc;
            local += acc;
        }
    }
    if (pool_mean) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0) red[warp] = local;
        __syncthreads();
        if (threadIdx.x == 0) {
            float tot = 0.0f;
            for (int i = 0; i < 8; ++i) tot += red[i];
            pool_mean[img * g.m + ch] = tot / (g.oh * g.ow);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// squeeze-excite gate: one block per image
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) se_gate_kernel(const T* __restrict__ pooled, const T* __restrict__ w1,
                                                      const T* __restrict__ b1, const T* __restrict__ w2,
                                                      const T* __restrict__ b2, T* __restrict__ gate, int c, int r) {
    extern __shared__ float sm[];  // pooled[c] then hidden[r]
    float* ps = sm;
    float* hs = sm + c;
    const int64_t img = blockIdx.x;
    for (int i = threadIdx.x; i < c; i += blockDim.x) ps[i] = ldv(pooled + img * c + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int rr = warp; rr < r; rr += nw) {
        float s = 0.0f;
        for (int i = lane; i < c; i += 32) s = fmaf(ldv(w1 + static_cast<int64_t>(rr) * c + i), ps[i], s);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            s += b1 ? ldv(b1 + rr) : 0.0f;
            hs[rr] = s * sigmoidf_(s);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < c; i += blockDim.x) {
        float s = b2 ? ldv(b2 + i) : 0.0f;
        for (int rr = 0; rr < r; ++rr) s = fmaf(ldv(w2 + static_cast<int64_t>(i) * r + rr), hs[rr], s);
        stv(gate + img * c + i, sigmoidf_(s));
    }
}

template <typename T>
int launch_direct(const b200ml_conv_params* p, const ConvGeom& g, cudaStream_t s) {
    const int mg = g.m / g.group;
    const int64_t npix = static_cast<int64_t>(g.n) * g.oh * g.ow;
    const int64_t gy = static_cast<int64_t>(g.group) * ceil_div(mg, MT);
    B200ML_REQUIRE(gy <= 65535, "conv: too many output-channel blocks");
    const dim3 grid((unsigned)ceil_div(npix, 256), (unsigned)gy);
    if (g.kh == 3 && g.kw == 3)
        conv_direct_kernel<T, 3><<<grid, 256, 0, s>>>((const T*)p->x, (const T*)p->weight, (const T*)p->bias, (const T*)p->gate,
                                                      (const T*)p->residual, (T*)p->y, g);
    else
        conv_direct_kernel<T, 0><<<grid, 256, 0, s>>>((const T*)p->x, (const T*)p->weight, (const T*)p->bias, (const T*)p->gate,
                                                      (const T*)p->residual, (T*)p->y, g);
    return check_launch("conv_direct");
}

}  // namespace

// Tries the specialised kernels; *launched says whether one ran, *pooled whether it also wrote the pool.
static int conv2d_fast(const b200ml_ctx* ctx, const b200ml_conv_params* p, const ConvGeom& g, cudaStream_t s, bool* launched,
                       bool* pooled) {
    *launched = false;
    *pooled = false;
    if (p->dtype != B200ML_F32) return B200ML_OK;
    if (conv1x1_tensor_core_applies(ctx, p)) {  // 1x1, stride 1: the tensor-core kernel (3 x TF32), HBM-bound
        *launched = true;
        return conv1x1_tensor_core(ctx, p, s);
    }
    if (conv_igemm_applies(ctx, p, g.oh, g.ow)) {  // k x k, stride 1, group 1: implicit GEMM on the tensor core (3 x TF32)
        *launched = true;
        return conv_igemm(ctx, p, g.oh, g.ow, s);
    }
    const bool unit = p->stride_h == 1 && p->stride_w == 1 && p->dil_h == 1 && p->dil_w == 1;
    const bool nopad = !p->pad_top && !p->pad_left && !p->pad_bottom && !p->pad_right;
    const int64_t hw = p->h * p->w;
    const float *x = (const float*)p->x, *w = (const float*)p->weight, *b = (const float*)p->bias,
                *gt = (const float*)p->gate, *r = (const float*)p->residual;
    float* y = (float*)p->y;
    if (unit && nopad && p->group == 1 && p->kh == 1 && p->kw == 1 && hw % 4 == 0 && aligned16(x) && aligned16(y) &&
        (!r || aligned16(r))) {
        const int p4 = (int)(hw / 4);
        const int64_t total4 = p->n * (int64_t)p4;
        const int64_t gx64 = ceil_div(total4, 128);
        if (gx64 < (1ll << 31)) {
            const unsigned gx = (unsigned)gx64;
            const int c = (int)p->c, m = (int)p->m;
            if (c <= 32) {
                const int cp = c <= 4 ? 4 : (c <= 8 ? 8 : (c <= 16 ? 16 : (c <= 24 ? 24 : 32)));
                const size_t sm = (size_t)m * cp * sizeof(float);
                if (sm <= 48 * 1024) {
                    // One share of output channels (gridDim.y == 1): sharing them out over blockIdx.y, which the kernel
                    // supports, was measured slower (145.8 vs 132.3 us for 24 -> 144 channels at 112 x 112 x 64 images)
                    const dim3 gxy(gx, 1u);
                    switch (cp) {
                        case 4: pointwise_x_kernel<4><<<gxy, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                        case 8: pointwise_x_kernel<8><<<gxy, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                        case 16: pointwise_x_kernel<16><<<gxy, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                        case 24: pointwise_x_kernel<24><<<gxy, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                        default: pointwise_x_kernel<32><<<gxy, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                    }
                    *launched = true;
                    return check_launch("pointwise_x");
                }
            }
            const int mp = m <= 8 ? 8 : (m <= 16 ? 16 : (m <= 24 ? 24 : 32));
            const size_t sm = (((size_t)c * mp + 3) & ~(size_t)3) * sizeof(float) + ACC_RING_BYTES;  // weights + the X rings
            if (sm <= ACC_SMEM_LIMIT) {
                static const bool opted_in = [] {  // dynamic shared memory above 48 KB has to be asked for, once per kernel
                    bool ok = true;
                    ok &= cudaFuncSetAttribute(pointwise_acc_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ACC_SMEM_LIMIT) == cudaSuccess;
                    ok &= cudaFuncSetAttribute(pointwise_acc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ACC_SMEM_LIMIT) == cudaSuccess;
                    ok &= cudaFuncSetAttribute(pointwise_acc_kernel<24>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ACC_SMEM_LIMIT) == cudaSuccess;
                    ok &= cudaFuncSetAttribute(pointwise_acc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ACC_SMEM_LIMIT) == cudaSuccess;
                    return ok;
                }();
                if (!opted_in && sm > 48 * 1024) return fail(B200ML_ERR_CUDA, "conv: cannot reserve %zu bytes of shared memory", sm);
                const dim3 grid(gx, (unsigned)ceil_div(m, mp));
                switch (mp) {
                    case 8: pointwise_acc_kernel<8><<<grid, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                    case 16: pointwise_acc_kernel<16><<<grid, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                    case 24: pointwise_acc_kernel<24><<<grid, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                    default: pointwise_acc_kernel<32><<<grid, 128, sm, s>>>(x, w, b, gt, r, y, total4, p4, c, m, p->act); break;
                }
                *launched = true;
                return check_launch("pointwise_acc");
            }
        }
    }
    if (unit && p->group == p->c && p->m == p->c && !gt && !r && p->kh * p->kw <= 64) {
        const size_t sm = (size_t)(g.oh + p->kh - 1) * (g.ow + p->kw - 1) * sizeof(float);
        if (sm <= 40 * 1024 && p->n * p->c < (1ll << 31)) {
            const bool pad1 = p->pad_top == 1 && p->pad_left == 1 && p->pad_bottom == 1 && p->pad_right == 1;
            if (p->kh == 3 && p->kw == 3 && pad1 && p->w % 4 == 0 && p->w >= 8 && p->w <= 64 && aligned16(x) && aligned16(y)) {
                const int64_t planes = p->n * p->c;
                depthwise3x3_quad_kernel<<<(unsigned)ceil_div(planes, 4), 128, 0, s>>>(x, w, b, y, p->pool_sum, g, planes);
            } else if (p->kh == 3 && p->kw == 3 && g.ow <= 64) depthwise3x3_kernel<<<(unsigned)(p->n * p->c), 256, 0, s>>>(x, w, b, y, p->pool_sum, g);
            else depthwise_plane_kernel<<<(unsigned)(p->n * p->c), 256, sm, s>>>(x, w, b, y, p->pool_sum, g);
            *launched = true;
            *pooled = true;
            return check_launch("depthwise_plane");
        }
    }
    return B200ML_OK;
}

int conv2d(const b200ml_ctx* ctx, const b200ml_conv_params* p, cudaStream_t s) {
    B200ML_REQUIRE(p->group >= 1 && p->c % p->group == 0 && p->m % p->group == 0, "conv: channels not divisible by group");
    B200ML_REQUIRE(p->stride_h >= 1 && p->stride_w >= 1 && p->dil_h >= 1 && p->dil_w >= 1, "conv: bad stride or dilation");
    B200ML_REQUIRE(p->kh >= 1 && p->kw >= 1, "conv: empty kernel");
    const int64_t eh = p->h + p->pad_top + p->pad_bottom - p->dil_h * (p->kh - 1) - 1;
    const int64_t ew = p->w + p->pad_left + p->pad_right - p->dil_w * (p->kw - 1) - 1;
    B200ML_REQUIRE(eh >= 0 && ew >= 0, "conv: kernel larger than the padded input");
    const int64_t oh = eh / p->stride_h + 1, ow = ew / p->stride_w + 1;
    if (p->n == 0 || p->m == 0) return B200ML_OK;
    ConvGeom g{(int32_t)p->n, (int32_t)p->c, (int32_t)p->h, (int32_t)p->w, (int32_t)p->m, (int32_t)p->kh,
               (int32_t)p->kw, (int32_t)p->stride_h, (int32_t)p->stride_w, (int32_t)p->pad_top, (int32_t)p->pad_left,
               (int32_t)p->dil_h, (int32_t)p->dil_w, (int32_t)p->group, (int32_t)oh, (int32_t)ow, p->act};
    bool launched = false, pooled = false;
    int rc = conv2d_fast(ctx, p, g, s, &launched, &pooled);
    if (rc) return rc;
    if (!launched) {
        rc = p->dtype == B200ML_F32 ? launch_direct<float>(p, g, s) : launch_direct<__half>(p, g, s);
        if (rc) return rc;
    }
    if (p->pool_sum && !pooled) {
        // no specialised kernel wrote the pool: the mean of every output plane, in the tensors' own type
        return reduce(ctx, p->dtype, B200ML_RED_MEAN, p->y, p->pool_sum, p->n * p->m, oh * ow, 1, s);
    }
    return B200ML_OK;
}

// Which tensor-core kernel (if any) takes this convolution: 1 = the 1x1 kernel, 2 = the implicit GEMM, 0 = neither.
static int conv_tensor_core_kind(const b200ml_ctx* ctx, const b200ml_conv_params* p, int64_t* ow_out) {
    if (p->group < 1 || p->stride_h < 1 || p->stride_w < 1 || p->dil_h < 1 || p->dil_w < 1 || p->kh < 1 || p->kw < 1) return 0;
    const int64_t eh = p->h + p->pad_top + p->pad_bottom - p->dil_h * (p->kh - 1) - 1;
    const int64_t ew = p->w + p->pad_left + p->pad_right - p->dil_w * (p->kw - 1) - 1;
    if (eh < 0 || ew < 0 || p->n == 0 || p->m == 0) return 0;
    const int64_t oh = eh / p->stride_h + 1, ow = ew / p->stride_w + 1;
    *ow_out = ow;
    // the pointers only enter through their alignment, and prepacking is asked with the tensors the calls will use or none
    b200ml_conv_params q = *p;
    if (!q.x) q.x = reinterpret_cast<const void*>(uintptr_t(256));
    if (!q.y) q.y = reinterpret_cast<void*>(uintptr_t(256));
    if (conv1x1_tensor_core_applies(ctx, &q)) return 1;
    if (conv_igemm_applies(ctx, &q, oh, ow)) return 2;
    return 0;
}

int64_t conv_prepack_bytes(const b200ml_ctx* ctx, const b200ml_conv_params* p) {
    int64_t ow = 0;
    const int kind = conv_tensor_core_kind(ctx, p, &ow);
    return kind == 1 ? conv1x1_pack_bytes(p) : (kind == 2 ? conv_igemm_pack_bytes(p, ow) : 0);
}

int conv_prepack(const b200ml_ctx* ctx, const b200ml_conv_params* p, void* packed, cudaStream_t s) {
    int64_t ow = 0;
    const int kind = conv_tensor_core_kind(ctx, p, &ow);
    B200ML_REQUIRE(kind != 0, "conv_prepack: this convolution takes its weights as they are (b200ml_conv_prepack_bytes returns 0)");
    B200ML_REQUIRE(packed && aligned16(packed) && p->weight, "conv_prepack: the packed buffer must be 16-byte aligned device memory, the weights given");
    return kind == 1 ? conv1x1_pack(ctx, p, packed, s) : conv_igemm_pack(ctx, p, ow, packed, s);
}

int se_gate(const b200ml_ctx*, int dtype, const void* pooled, const void* w1, const void* b1, const void* w2,
            const void* b2, void* gate, int64_t n, int64_t c, int64_t r, cudaStream_t s) {
    if (n == 0 || c == 0) return B200ML_OK;
    const size_t sm = (size_t)(c + r) * sizeof(float);
    B200ML_REQUIRE(sm <= 48 * 1024, "se_gate: too many channels");
    if (dtype == B200ML_F16)
        se_gate_kernel<__half><<<(unsigned)n, 256, sm, s>>>((const __half*)pooled, (const __half*)w1, (const __half*)b1,
                                                           (const __half*)w2, (const __half*)b2, (__half*)gate, (int)c, (int)r);
    else
        se_gate_kernel<float><<<(unsigned)n, 256, sm, s>>>((const float*)pooled, (const float*)w1, (const float*)b1,
                                                          (const float*)w2, (const float*)b2, (float*)gate, (int)c, (int)r);
    return check_launch("se_gate");
}

}  // namespace b200ml
