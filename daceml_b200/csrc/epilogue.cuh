// The element-wise tail shared by the GEMM and convolution kernels:
//   out = act(alpha * acc + bias_scale * bias[n]) + residual_scale * residual[m, n]
// All math is fp32; erf / exp are the full-precision libm versions (the reference strips
// --use_fast_math because it produced NaNs in BERT, daceml/__init__.py:13-19).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/daceml_b200.h"

namespace b200ml {

struct EpilogueParams {
    int32_t flags;
    float alpha, bias_scale, residual_scale;
};

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float apply_act(float v, int32_t flags) {
    if (flags & B200ML_EPI_RELU) v = fmaxf(v, 0.0f);
    if (flags & B200ML_EPI_GELU) v = gelu_erf(v);
    if (flags & B200ML_EPI_SWISH) v = v * sigmoidf_(v);
    return v;
}

// Activation of the convolution kernels.  Swish goes through one MUFU.EX2 and one MUFU.RCP (relative error about
// 1e-6, against the 1e-4 the fp32 configurations allow): the libm expf + division cost more instructions than the
// nine multiply-adds of a depthwise tap.  No NaN for any finite input: exp2 saturates to +inf or 0, 1 / inf = 0.
__device__ __forceinline__ float conv_act(float v, int act) {
    if (act & B200ML_EPI_RELU) return fmaxf(v, 0.0f);
    if (act & B200ML_EPI_SWISH) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.44269504088896340736f * v));
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
        return v * r;
    }
    if (act & B200ML_EPI_GELU) return gelu_erf(v);
    return v;
}


__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 q;
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return q;
}

// GELU (erf form) for fp16 outputs.  With z = |x| / sqrt(2) and e = erfc(z) = 2^(-q(z)), q a fitted degree-5
// polynomial (|erf error| < 7e-7, one MUFU.EX2): Phi(x) = 1 - e/2 for x >= 0 and e/2 for x < 0, hence
// gelu(x) = max(x, 0) - |x| e / 2 - no cancellation on the negative side, no select.
__device__ __forceinline__ float gelu_erf_fast(float x) {
    const float z = fabsf(x) * 0.70710678118654752440f;
    float q = fmaf(z, 0.0029446918051689863f, -0.02959194779396057f);
    q = fmaf(z, q, 0.1486678570508957f);
    q = fmaf(z, q, 0.9185084104537964f);
    q = fmaf(z, q, 1.6278891563415527f);
    q *= z;
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-q));
    return fmaf(-0.70710678118654752440f * z, e, fmaxf(x, 0.0f));  // |x| / 2 = z / sqrt(2)
}

// The same form on two values at a time in half precision, for results that are stored as fp16 anyway: half the
// instructions per value (the GELU of an FFN epilogue is 33 M values per layer).  The pre-activation is rounded to fp16
// first, which moves the result by at most gelu'(x) <= 1.13 fp16 steps of x; the polynomial and the exponential carry
// about one more step each on the small term |x| e / 2, and the last subtraction rounds like the store would.
__device__ __forceinline__ __half2 gelu_erf_fast_h2(__half2 x) {
    const __half2 ax = __habs2(x);
    const __half2 z = __hmul2(ax, __float2half2_rn(0.70710678118654752440f));
    __half2 q = __hfma2(z, __float2half2_rn(0.0029446918051689863f), __float2half2_rn(-0.02959194779396057f));
    q = __hfma2(z, q, __float2half2_rn(0.1486678570508957f));
    q = __hfma2(z, q, __float2half2_rn(0.9185084104537964f));
    q = __hfma2(z, q, __float2half2_rn(1.6278891563415527f));
    q = __hmul2(q, z);
    const __half2 e = h2exp2(__hneg2(q));
    return __hfma2(__hmul2(ax, __float2half2_rn(-0.5f)), e, __hmax2(x, __float2half2_rn(0.0f)));
}

// Eight fp32 pre-activations -> eight fp16 GELU values.
__device__ __forceinline__ uint4 gelu_pack8(const float (&f)[8]) {
    uint4 q;
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = gelu_erf_fast_h2(__floats2half2_rn(f[2 * i], f[2 * i + 1]));
    return q;
}

// Activation for results that are stored as fp16: GELU through the one-MUFU form above.
__device__ __forceinline__ float apply_act_f16(float v, int32_t flags) {
    if (flags & B200ML_EPI_RELU) v = fmaxf(v, 0.0f);
    if (flags & B200ML_EPI_GELU) v = gelu_erf_fast(v);
    if (flags & B200ML_EPI_SWISH) v = v * sigmoidf_(v);
    return v;
}

// Residual / bias packets of one 32-column chunk, fetched before the accumulator arrives.
struct EpiloguePrefetch {
    uint4 res[4];
    uint4 bias[4];
};

__device__ __forceinline__ void epilogue_prefetch_32(const EpilogueParams& ep, EpiloguePrefetch& pf, const __half* r_row,
                                                     const __half* bias, int col0, int n, bool vec) {
    if (!(vec && n - col0 >= 32)) return;
    if ((ep.flags & B200ML_EPI_RESIDUAL) && r_row != nullptr) {
#pragma unroll
        for (int g = 0; g < 4; ++g) pf.res[g] = __ldg(reinterpret_cast<const uint4*>(r_row + col0 + g * 8));
    }
    if ((ep.flags & B200ML_EPI_BIAS) && bias != nullptr) {
#pragma unroll
        for (int g = 0; g < 4; ++g) pf.bias[g] = __ldg(reinterpret_cast<const uint4*>(bias + col0 + g * 8));
    }
}

// Finishes 32 consecutive columns of one output row held as raw fp32 bits in r and returns them as four
// packets of eight fp16 values (the caller stages them in shared memory for a bulk tensor store).  The
// bias / residual packets come from epilogue_prefetch_32; every branch on ep.flags is warp-uniform.
__device__ __forceinline__ void epilogue_pack_32(const EpilogueParams& ep, const uint32_t (&r)[32],
                                                 const EpiloguePrefetch& pf, bool has_bias, bool has_res, uint4 (&out)[4]) {
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (ep.alpha != 1.0f) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= ep.alpha;
    }
    if (has_bias) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float b[8];
            unpack8(pf.bias[g], b);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[g * 8 + j] = fmaf(ep.bias_scale, b[j], v[g * 8 + j]);
        }
    }
    if ((ep.flags & B200ML_EPI_GELU) && !has_res) {  // the FFN form: GELU on pairs in half precision, straight into the packets
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[g * 8 + j];
            out[g] = gelu_pack8(o);
        }
        return;
    }
    if (ep.flags & B200ML_EPI_GELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = gelu_erf_fast(v[j]);
    } else if (ep.flags & B200ML_EPI_RELU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
    } else if (ep.flags & B200ML_EPI_SWISH) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = v[j] * sigmoidf_(v[j]);
    }
    if (has_res) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float q[8];
            unpack8(pf.res[g], q);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[g * 8 + j] = fmaf(ep.residual_scale, q[j], v[g * 8 + j]);
        }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[g * 8 + j];
        out[g] = pack8(o);
    }
}

// Finishes 32 consecutive columns [col0, col0 + 32) of one output row held as raw fp32 bits in r.
// Every branch on ep.flags is warp-uniform; the per-element work is alpha, bias, activation,
// residual, one fp16 conversion.
__device__ __forceinline__ void epilogue_store_32(const EpilogueParams& ep, const uint32_t (&r)[32],
                                                  const EpiloguePrefetch& pf, __half* c_row, const __half* r_row,
                                                  const __half* bias, int col0, int n, bool vec) {
    const int valid = n - col0 < 32 ? n - col0 : 32;
    const bool has_bias = (ep.flags & B200ML_EPI_BIAS) && bias != nullptr;
    const bool has_res = (ep.flags & B200ML_EPI_RESIDUAL) && r_row != nullptr;
    if (vec && valid == 32) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (ep.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= ep.alpha;
        }
        if (has_bias) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float b[8];
                unpack8(pf.bias[g], b);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[g * 8 + j] = fmaf(ep.bias_scale, b[j], v[g * 8 + j]);
            }
        }
        if (ep.flags & B200ML_EPI_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_erf_fast(v[j]);
        } else if (ep.flags & B200ML_EPI_RELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        } else if (ep.flags & B200ML_EPI_SWISH) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = v[j] * sigmoidf_(v[j]);
        }
        if (has_res) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float q[8];
                unpack8(pf.res[g], q);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[g * 8 + j] = fmaf(ep.residual_scale, q[j], v[g * 8 + j]);
            }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = v[g * 8 + j];
            *reinterpret_cast<uint4*>(c_row + col0 + g * 8) = pack8(o);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (j < valid) {
                float v = ep.alpha * __uint_as_float(r[j]);
                if (has_bias) v = fmaf(ep.bias_scale, __half2float(bias[col0 + j]), v);
                v = apply_act(v, ep.flags);
                if (has_res) v = fmaf(ep.residual_scale, __half2float(r_row[col0 + j]), v);
                c_row[col0 + j] = __float2half_rn(v);
            }
        }
    }
}

}  // namespace b200ml
