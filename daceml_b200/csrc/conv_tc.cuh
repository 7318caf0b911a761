// What the tensor-core convolution kernels share: the tf32 instruction descriptor and MMA, the shared-memory descriptor
// of an MN-major 32-bit operand, the hi / lo split behind the 3 x TF32 products, and the epilogue turn that finishes two
// 8-channel units of 32 pixels.
#pragma once

#include "gemm_common.cuh"

namespace b200ml {
namespace convtc {

constexpr int PW_BM = 128;  // pixels per accumulator = UMMA M

// D = f32, A = B = tf32, A MN-major (bit 15), B K-major or MN-major (bit 16), N >> 3 in [17,23), M >> 4 in [24,29)
__host__ __device__ constexpr uint32_t pw_idesc(uint32_t npad, uint32_t b_mn_major = 0) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (b_mn_major << 16) | ((npad >> 3) << 17) | ((PW_BM >> 4) << 24);
}

__device__ __forceinline__ void pw_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory descriptor of an MN-major 32-bit operand: the 128-byte swizzle with 32-byte atoms (layout type 1; the
// only layout tcgen05.mma takes for MN-major tf32).  Atoms are 128 bytes (32 elements along MN) x 4 K-rows; `lbo` is
// the distance between atoms along MN, `sbo` between 4-row groups along K.
__device__ __forceinline__ uint64_t make_smem_desc_sw128_base32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= 1ull << 61;
    return d;
}

__device__ __forceinline__ float4 ld_shared_v4(uint32_t saddr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, float4 v) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t saddr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void st_shared_f32(uint32_t saddr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(saddr), "f"(v) : "memory");
}

// hi = the leading TF32 bits of v (sign, exponent, 10 mantissa bits: exactly representable), lo = v - hi (exact in fp32,
// |lo| < 2^-10 |v|).  Infinities and NaNs stay in hi with lo = 0.
__device__ __forceinline__ void split_tf32(float v, float& hi, float& lo) {
    hi = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    lo = fabsf(v) < __int_as_float(0x7f800000) ? v - hi : 0.0f;
}

// The activation as a template argument: the sixteen values of a turn then form one straight-line block that the
// compiler can interleave; a run-time test per value would cut it into sixteen dependent pieces.
template <int ACT>
__device__ __forceinline__ float pw_act(float v) {
    if (ACT == B200ML_EPI_RELU) return fmaxf(v, 0.0f);
    if (ACT == B200ML_EPI_SWISH || ACT == B200ML_EPI_GELU) return conv_act(v, ACT);
    return v;
}

// Finishes two 8-channel units of 32 pixels: activation, residual, and the values into the warp's two staging boxes
// ([8 channels][32 pixels] each; lane = pixel, so every store instruction fills one 128-byte row without conflicts).
template <int ACT, bool RES>
__device__ __forceinline__ void pw_finish_turn(const uint32_t (&r)[2][8], const float (&rv)[2][8], uint32_t stg_lane) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float va = pw_act<ACT>(__uint_as_float(r[0][j]));
        float vb = pw_act<ACT>(__uint_as_float(r[1][j]));
        if (RES) va += rv[0][j], vb += rv[1][j];
        st_shared_f32(stg_lane + j * 128, va);
        st_shared_f32(stg_lane + 1024 + j * 128, vb);
    }
}

}  // namespace convtc
}  // namespace b200ml
