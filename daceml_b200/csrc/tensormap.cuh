// Tensor maps, encoded once per distinct (address, extents, strides, box) and then reused.
//
// cuTensorMapEncodeTiled costs a few microseconds of host time; a GEMM launch needs three or four maps, a fused
// attention three.  Under CUDA-graph replay that cost is paid once at capture, but eager calls (the donnx frontend, a
// DaceModule without cuda_graph) would pay it on every launch.  Models call the same operands again and again, so the
// encoded 128-byte maps are kept in a small per-thread table keyed by everything the encoding depends on.
#pragma once

#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace b200ml {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A rank-4 tiled map with unit element strides, no interleave, 128-byte swizzle, 256-byte L2 promotion and no fill
// value: the only form the kernels of this library use.  Returns the driver's result code.
// `swizzle`: CU_TENSOR_MAP_SWIZZLE_128B for every operand but an MN-major 32-bit one, which tcgen05.mma reads in the
// 128-byte swizzle with 32-byte atoms (CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B).
CUresult encode_tiled_cached(const b200ml_ctx* ctx, CUtensorMap* out, CUtensorMapDataType dtype, const void* base,
                             const cuuint64_t dims[4], const cuuint64_t strides[3], const cuuint32_t box[4],
                             CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

// Hits and misses of the calling thread's table since the library was loaded (for tests and tuning).
void tensormap_cache_counters(int64_t* hits, int64_t* misses);

}  // namespace b200ml
