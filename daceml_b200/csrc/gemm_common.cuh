// Pieces shared by the one-CTA and the CTA-pair tcgen05 GEMM kernels.
#pragma once

#include "common.cuh"
#include "ptx.cuh"
#include "epilogue.cuh"
#include "tensormap.cuh"

namespace b200ml {
namespace gemm {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 fp16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int EPI_WARPS = 8;  // two per TMEM lane quarter, each taking half of the tile's columns
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;

struct GemmArgs {
    int32_t m, n, k;
    int32_t tiles_m, tiles_n, num_tiles;
    int32_t batch_inner;
    int32_t epilogue;
    // 0 when the operand is broadcast over that batch loop (its TMA coordinate stays 0)
    int32_t a_use_inner, a_use_outer, b_use_inner, b_use_outer;
    int64_t ldc, c_so, c_si;
    int64_t ldr, r_so, r_si;
    float alpha, bias_scale, residual_scale;
    int32_t vec_ok;  // C (and residual) rows are 16-byte aligned
    int32_t b_early;    // B is a constant of the stream: its first pipeline stages are fetched before griddepcontrol.wait
    int32_t tma_store;  // the kernel got a tensor map of C: finished tiles leave through shared memory and bulk stores
    __half* c;
    const __half* bias;
    const __half* residual;
    int32_t* status;
    long long* trace;  // per-CTA cycle counters, only written when built with B200ML_TRACE
};

#ifdef B200ML_TRACE
#define TRACE_T0() const long long _t0 = clock64()
#define TRACE_ADD(var) var += clock64() - _t0
#else
#define TRACE_T0()
#define TRACE_ADD(var)
#endif

// rank-4 fp16 tensor map {inner, rows, batch_inner, batch_outer} with a 128-byte-swizzled box.
inline int make_tmap(const b200ml_ctx* ctx, CUtensorMap* out, const void* base, int64_t inner, int64_t rows, int64_t ld,
              int64_t n_inner, int64_t s_inner, int64_t n_outer, int64_t s_outer, int box_inner, int box_rows,
              const char* what) {
    if (!aligned16(base)) return fail(B200ML_ERR_UNSUPPORTED, "gemm f16: %s base is not 16-byte aligned", what);
    if (ld % 8 != 0) return fail(B200ML_ERR_UNSUPPORTED, "gemm f16: %s leading dimension %lld is not a multiple of 8", what, (long long)ld);
    const bool use_i = n_inner > 1 && s_inner != 0;
    const bool use_o = n_outer > 1 && s_outer != 0;
    if ((use_i && s_inner % 8 != 0) || (use_o && s_outer % 8 != 0))
        return fail(B200ML_ERR_UNSUPPORTED, "gemm f16: %s batch stride is not a multiple of 8 elements", what);
    const uint64_t row_bytes = static_cast<uint64_t>(ld) * 2;
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(use_i ? n_inner : 1), static_cast<cuuint64_t>(use_o ? n_outer : 1)};
    // A size-1 dimension still needs a legal stride (non-zero multiple of 16 bytes).
    const uint64_t dummy = row_bytes * static_cast<uint64_t>(rows);
    cuuint64_t strides[3] = {row_bytes, use_i ? static_cast<uint64_t>(s_inner) * 2 : dummy,
                             use_o ? static_cast<uint64_t>(s_outer) * 2 : dummy};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows), 1, 1};
    if (!ctx->encode_tiled) return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUresult r = encode_tiled_cached(ctx, out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base, dims, strides, box);
    if (r != CUDA_SUCCESS)
        return fail(B200ML_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d (dims %llu x %llu, ld %lld)", what,
                    (int)r, (unsigned long long)dims[0], (unsigned long long)dims[1], (long long)ld);
    return B200ML_OK;
}


}  // namespace gemm
}  // namespace b200ml
