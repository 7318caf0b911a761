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
    DEV_BAD_INDEX = 5,  // Gather met an index outside its axis
    DEV_TIMEOUT_PROBE = 6,  // the wait probe's barrier was (as intended) never completed
    DEV_TIMEOUT_PEER = 7,   // a rank's all-gather kernel gave up waiting for a peer's flag
};

struct b200ml_ctx {
    int device = 0;
    int sm_count = 0;
    void* workspace = nullptr;
    int64_t workspace_bytes = 0;
    int32_t* status_dev = nullptr;  // one word in device memory
    void* encode_tiled = nullptr;   // cuTensorMapEncodeTiled, resolved through the runtime
    void* mem_get_address_range = nullptr;  // cuMemGetAddressRange, likewise
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

// Programmatic dependent launch: a kernel launched through launch_pdl() may start while its
// predecessor in the stream is still draining, run its set-up (barrier init, TMEM allocation,
// descriptor prefetch) and then block in pdl_wait() until the predecessor has completed and its
// writes are visible.  B200ML_PDL=0 turns the attribute off (plain stream order).
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Makes the context's device current for the duration of a call.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) {
            switched = cudaSetDevice(dev) == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace b200ml

#ifdef __CUDACC__
// Lets the next kernel in the stream begin its set-up.  Issued first thing by every CTA, so a
// dependent grid can only start once all CTAs of this grid have been scheduled.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
// Blocks until every kernel before this one in the stream has completed and flushed its writes.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

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
