// Shared host-side plumbing of libdaceml_b200: context, status codes, launch accounting.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <atomic>

#include "../../include/daceml_b200.h"

// Device-side status codes written to the context's status word by kernels whose bounded
// waits ran out.  0 means "no error".
enum : int32_t {
    DEV_OK = 0,
    DEV_TIMEOUT_PRODUCER = 1,  // TMA producer gave up waiting for a free stage
    DEV_TIMEOUT_MMA = 2,       // MMA issuer gave up waiting for operands or a free accumulator
    DEV_TIMEOUT_EPILOGUE = 3,  // epilogue gave up waiting for an accumulator
    DEV_TIMEOUT_ATTN = 4,
};

struct b200ml_ctx {
    int device = 0;
    int sm_count = 0;
    void* workspace = nullptr;
    int64_t workspace_bytes = 0;
    int32_t* status_dev = nullptr;  // one word in device memory
    void* encode_tiled = nullptr;   // cuTensorMapEncodeTiled, resolved through the runtime
};

namespace b200ml {

void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
extern std::atomic<int64_t> g_launches;

inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Checks the launch itself (configuration errors); does not synchronise.
inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200ML_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    count_launch();
    return B200ML_OK;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace b200ml

#define B200ML_REQUIRE(cond, ...)                                         \
    do {                                                                  \
        if (!(cond)) return b200ml::fail(B200ML_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define B200ML_CUDA(call)                                                                          \
    do {                                                                                           \
        cudaError_t _e = (call);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return b200ml::fail(B200ML_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(_e)); \
    } while (0)
