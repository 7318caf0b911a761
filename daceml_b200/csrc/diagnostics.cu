// Diagnostics: the bounded-wait path of the kernels, run on purpose.
//
// Every device-side wait in this library (ptx::mbar_wait) gives up after a wall-clock limit, records a code in the
// context's status word and lets the kernel end normally; the host reads the word with b200ml_ctx_device_status.
// b200ml_wait_probe runs exactly that sequence with a short limit: one CTA initialises an mbarrier that expects one
// arrival, nobody ever arrives, the wait runs out, the code is recorded, the CTA reaches its closing barrier and
// returns.  Nothing traps, nothing is left waiting, the context stays usable.
#include "common.cuh"
#include "ptx.cuh"

namespace b200ml {
namespace {

__global__ void __launch_bounds__(128) wait_probe_kernel(int32_t* status, uint64_t limit_ns, uint32_t* waited_us) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint64_t t0 = ptx::global_timer_ns();
        const bool completed = ptx::mbar_wait(&bar, 0, limit_ns);  // phase 0 never completes: no thread arrives
        if (!completed) atomicExch(status, DEV_TIMEOUT_PROBE);
        if (waited_us) *waited_us = static_cast<uint32_t>((ptx::global_timer_ns() - t0) / 1000u);
    }
    __syncthreads();  // the other warps wait here, as the epilogue warps of a GEMM wait for their issuer
}

}  // namespace
}  // namespace b200ml

extern "C" int b200ml_wait_probe(b200ml_ctx* ctx, int64_t limit_ns, uint32_t* waited_us, b200ml_stream stream) {
    using namespace b200ml;
    if (ctx == nullptr) return fail(B200ML_ERR_INVALID, "wait_probe: null context");
    B200ML_REQUIRE(limit_ns > 0 && limit_ns <= 100ll * 1000 * 1000, "wait_probe: the limit must be between 1 ns and 100 ms");
    DeviceGuard guard(ctx->device);
    wait_probe_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(ctx->status_dev, static_cast<uint64_t>(limit_ns), waited_us);
    return check_launch("wait_probe");
}
